// Loss-side and front-end kernels: vocabulary cross-entropy with fused
// gradient, flow-matching velocity MSE with fused gradient, exact GELU,
// column sums for bias gradients and the 2-D rotary embedding of the pixel
// patch front-end.
//
// References: per-token weighted CE training/sensenovalm/model/losses/ce_loss.py:19-84
// and ops/cross_entropy.py:159-343; flow-matching loss
// training/sensenovavl/model/sensenovavl_moe_chat/modeling_sensenovavl_chat_mot.py:1403-1480;
// patch front-end src/sensenova_u1/models/neo_unify/modeling_neo_vit.py:12-204.
#include "host_common.h"
#include "sm100_common.cuh"

namespace snu1 {

__device__ __forceinline__ void unpack8f(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8f(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

// ---------------------------------------------------------------------------
// Cross-entropy over one row of logits per CTA; the logits are overwritten by
// their gradient  (softmax - onehot) * weight * grad_scale.
//   loss_out[0] += weight * (lse - logit[label]);  loss_out[1] += weight
//   loss_out[2] += (argmax == label)               loss_out[3] += 1 (valid rows)
// Rows with label < 0 get a zero gradient and contribute nothing.
// ---------------------------------------------------------------------------
constexpr int CE_THREADS = 512;

__global__ void __launch_bounds__(CE_THREADS)
    ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, long long ld, const int* __restrict__ labels,
                      const float* __restrict__ weights, float grad_scale, float* __restrict__ loss_out,
                      float* __restrict__ row_loss, int rows, int V) {
  __shared__ float s_max[CE_THREADS / 32], s_sum[CE_THREADS / 32];
  __shared__ int s_arg[CE_THREADS / 32];
  const int nvec = V / 8;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    uint4* lr = reinterpret_cast<uint4*>(logits + (long long)row * ld);
    const int label = labels[row];
    const float w = weights ? weights[row] : 1.f;
    if (label < 0 || label >= V) {
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int v = threadIdx.x; v < nvec; v += CE_THREADS) lr[v] = z;
      if (threadIdx.x == 0 && row_loss) row_loss[row] = 0.f;
      continue;
    }
    float mx = -INFINITY, sum = 0.f;
    int arg = 0;
    for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
      float f[8];
      unpack8f(lr[v], f);
      float cm = f[0];
      int ca = 0;
#pragma unroll
      for (int i = 1; i < 8; ++i)
        if (f[i] > cm) {
          cm = f[i];
          ca = i;
        }
      if (cm > mx) {
        sum *= __expf(mx - cm);
        mx = cm;
        arg = v * 8 + ca;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) sum += __expf(f[i] - mx);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, mx, o);
      const float os = __shfl_xor_sync(0xffffffffu, sum, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      const float nm = fmaxf(mx, om);
      sum = (mx == -INFINITY ? 0.f : sum * __expf(mx - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
      if (om > mx || (om == mx && oa < arg)) arg = oa;
      mx = nm;
    }
    __syncthreads();
    if (lane == 0) {
      s_max[warp] = mx;
      s_sum[warp] = sum;
      s_arg[warp] = arg;
    }
    __syncthreads();
    float gm = -INFINITY;
    int ga = 0;
#pragma unroll
    for (int i = 0; i < CE_THREADS / 32; ++i)
      if (s_max[i] > gm || (s_max[i] == gm && s_arg[i] < ga)) {
        gm = s_max[i];
        ga = s_arg[i];
      }
    float gs = 0.f;
#pragma unroll
    for (int i = 0; i < CE_THREADS / 32; ++i)
      gs += s_max[i] == -INFINITY ? 0.f : s_sum[i] * __expf(s_max[i] - gm);
    const float lse = gm + __logf(gs);
    const float tgt = __bfloat162float(logits[(long long)row * ld + label]);
    __syncthreads();  // everyone has read logits[label] before it is overwritten
    if (threadIdx.x == 0) {
      const float loss = lse - tgt;
      if (row_loss) row_loss[row] = loss;
      atomicAdd(loss_out + 0, w * loss);
      atomicAdd(loss_out + 1, w);
      atomicAdd(loss_out + 2, ga == label ? 1.f : 0.f);
      atomicAdd(loss_out + 3, 1.f);
    }
    const float gsc = w * grad_scale;
    const int lv = label >> 3, li = label & 7;
    for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
      float f[8];
      unpack8f(lr[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = __expf(f[i] - lse) * gsc;
      if (v == lv) f[li] -= gsc;
      lr[v] = pack8f(f);
    }
  }
}

// ---------------------------------------------------------------------------
// Flow-matching loss on x-prediction:  v_pred = (x_pred - z) / max(1 - t, eps),
// loss_row = mean_d (v_pred - v)^2 * w[row];  dx = 2 (v_pred - v) w / (D den) * grad_scale.
//   loss_out[0] += sum_rows loss_row ;  row_loss[row] = mean_d (v_pred - v)^2
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
    fm_loss_kernel(const __nv_bfloat16* __restrict__ x_pred, const float* __restrict__ z,
                   const float* __restrict__ v_tgt, const float* __restrict__ t,
                   const float* __restrict__ w, float t_eps, float grad_scale,
                   __nv_bfloat16* __restrict__ dx, float* __restrict__ loss_out,
                   float* __restrict__ row_loss, int rows, int D) {
  __shared__ float scratch[8];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float den = fmaxf(1.f - t[row], t_eps);
    const float wr = w[row];
    const float gsc = 2.f * wr * grad_scale / (den * (float)D);
    float acc = 0.f;
    const long long base = (long long)row * D;
    for (int c = threadIdx.x * 4; c < D; c += 256 * 4) {
      const uint2 xr = *reinterpret_cast<const uint2*>(x_pred + base + c);
      const float4 zz = *reinterpret_cast<const float4*>(z + base + c);
      const float4 vv = *reinterpret_cast<const float4*>(v_tgt + base + c);
      const float2 x01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xr.x));
      const float2 x23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xr.y));
      const float e0 = (x01.x - zz.x) / den - vv.x, e1 = (x01.y - zz.y) / den - vv.y;
      const float e2 = (x23.x - zz.z) / den - vv.z, e3 = (x23.y - zz.w) / den - vv.w;
      acc += e0 * e0 + e1 * e1 + e2 * e2 + e3 * e3;
      if (dx) {
        uint2 o;
        o.x = pack_bf16x2(e0 * gsc, e1 * gsc);
        o.y = pack_bf16x2(e2 * gsc, e3 * gsc);
        *reinterpret_cast<uint2*>(dx + base + c) = o;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float tot = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) tot += scratch[i];
      tot /= (float)D;
      if (row_loss) row_loss[row] = tot;
      atomicAdd(loss_out, tot * wr);
    }
  }
}

// ---------------------------------------------------------------------------
// exact (erf) GELU
// ---------------------------------------------------------------------------
__global__ void gelu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                long long nvec) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float f[8];
    unpack8f(reinterpret_cast<const uint4*>(x)[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = 0.5f * f[j] * (1.f + erff(f[j] * 0.70710678118654752f));
    reinterpret_cast<uint4*>(y)[i] = pack8f(f);
  }
}
__global__ void gelu_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                __nv_bfloat16* __restrict__ dx, long long nvec) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float f[8], g[8];
    unpack8f(reinterpret_cast<const uint4*>(x)[i], f);
    unpack8f(reinterpret_cast<const uint4*>(dy)[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float cdf = 0.5f * (1.f + erff(f[j] * 0.70710678118654752f));
      const float pdf = 0.3989422804014327f * __expf(-0.5f * f[j] * f[j]);
      g[j] = g[j] * (cdf + f[j] * pdf);
    }
    reinterpret_cast<uint4*>(dx)[i] = pack8f(g);
  }
}

// out[col] += sum_rows x[row][col]   (bias gradients)
__global__ void __launch_bounds__(256)
    colsum_kernel(const __nv_bfloat16* __restrict__ x, long long ld, float* __restrict__ out,
                  int rows, int cols, int rows_per_cta) {
  const int col = (blockIdx.x * 256 + threadIdx.x) * 2;
  if (col >= cols) return;
  const int r0 = blockIdx.y * rows_per_cta;
  const int r1 = min(rows, r0 + rows_per_cta);
  float a = 0.f, b = 0.f;
  for (int r = r0; r < r1; ++r) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(x + (long long)r * ld + col));
    a += v.x;
    b += v.y;
  }
  atomicAdd(out + col, a);
  atomicAdd(out + col + 1, b);
}

// ---------------------------------------------------------------------------
// 2-D rotary embedding of patch features: the first half of the channels turns
// with the column index, the second half with the row index; pairs are
// interleaved (2i, 2i+1); angle = pos * theta^(-2i/half).  inverse = backward.
// ---------------------------------------------------------------------------
__global__ void rope2d_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                              const int* __restrict__ pos_x, const int* __restrict__ pos_y,
                              const float* __restrict__ inv_freq, int rows, int C, int inverse) {
  const int half = C / 2, pairs = half / 2;
  const long long total = (long long)rows * (C / 2);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(i / (C / 2));
    const int p = (int)(i - (long long)row * (C / 2));  // pair index over the whole row
    const bool second = p >= pairs;
    const int fi = second ? p - pairs : p;
    const float ang = (float)(second ? pos_y[row] : pos_x[row]) * inv_freq[fi];
    float sn, cs;
    sincosf(ang, &sn, &cs);
    if (inverse) sn = -sn;
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(x + (long long)row * C + 2 * p);
    const float2 f = __bfloat1622float2(v);
    const float o0 = f.x * cs - f.y * sn, o1 = f.x * sn + f.y * cs;
    *reinterpret_cast<uint32_t*>(y + (long long)row * C + 2 * p) = pack_bf16x2(o0, o1);
  }
}

}  // namespace snu1

using namespace snu1;

SNU1_API int snu1_ce_fwd_bwd(void* logits, long long ld, const int* labels, const float* weights,
                             float grad_scale, float* loss_out, float* row_loss, int rows, int V,
                             void* stream) {
  if (V % 8 != 0 || ld % 8 != 0 || rows <= 0) {
    set_last_error("ce_fwd_bwd: V and ld must be multiples of 8 (V=%d)", V);
    return kHostBadArg;
  }
  const int grid = rows < 148 * 4 ? rows : 148 * 4;
  ce_fwd_bwd_kernel<<<grid, CE_THREADS, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)logits, ld, labels, weights, grad_scale, loss_out, row_loss, rows, V);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_fm_loss(const void* x_pred, const float* z, const float* v_tgt, const float* t,
                          const float* w, float t_eps, float grad_scale, void* dx, float* loss_out,
                          float* row_loss, int rows, int D, void* stream) {
  if (D % 4 != 0 || rows <= 0) {
    set_last_error("fm_loss: D must be a multiple of 4");
    return kHostBadArg;
  }
  const int grid = rows < 148 * 8 ? rows : 148 * 8;
  fm_loss_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x_pred, z, v_tgt, t, w,
                                                         t_eps, grad_scale, (__nv_bfloat16*)dx,
                                                         loss_out, row_loss, rows, D);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_gelu_fwd(const void* x, void* y, long long n, void* stream) {
  if (n % 8 != 0 || n <= 0) {
    set_last_error("gelu: element count must be a positive multiple of 8");
    return kHostBadArg;
  }
  const long long nvec = n / 8;
  const int grid = (int)((nvec + 255) / 256 < 148 * 16 ? (nvec + 255) / 256 : 148 * 16);
  gelu_fwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, nvec);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_gelu_bwd(const void* x, const void* dy, void* dx, long long n, void* stream) {
  if (n % 8 != 0 || n <= 0) {
    set_last_error("gelu: element count must be a positive multiple of 8");
    return kHostBadArg;
  }
  const long long nvec = n / 8;
  const int grid = (int)((nvec + 255) / 256 < 148 * 16 ? (nvec + 255) / 256 : 148 * 16);
  gelu_bwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x,
                                                          (const __nv_bfloat16*)dy, (__nv_bfloat16*)dx, nvec);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_colsum(const void* x, long long ld, float* out, int rows, int cols, void* stream) {
  if (cols % 2 != 0 || ld % 2 != 0 || rows <= 0) {
    set_last_error("colsum: cols and ld must be even");
    return kHostBadArg;
  }
  const int rows_per_cta = 256;
  dim3 grid((cols / 2 + 255) / 256, (rows + rows_per_cta - 1) / rows_per_cta);
  colsum_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ld, out, rows, cols,
                                                        rows_per_cta);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_rope2d(const void* x, void* y, const int* pos_x, const int* pos_y,
                         const float* inv_freq, int rows, int C, int inverse, void* stream) {
  if (C % 4 != 0 || rows <= 0) {
    set_last_error("rope2d: channel count must be a multiple of 4");
    return kHostBadArg;
  }
  const long long total = (long long)rows * (C / 2);
  const int grid = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  rope2d_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, pos_x,
                                                        pos_y, inv_freq, rows, C, inverse);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}
