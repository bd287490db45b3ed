// Memory-bound kernels of the MoT decoder layer: RMSNorm with per-branch gains,
// the q/k half-head RMSNorm fused with the three-axis rotary embedding, and
// SwiGLU; forward and backward.  All of them work on the packed row layout
// "generation rows | understanding rows", where every 128-row tile belongs to
// one branch (tile_group), so a branch switch never needs a gather or a concat
// (reference: training/sensenovalm/model/modeling_qwen3_moe_mot.py:323-369).
//
// Math references: RMSNorm src/sensenova_u1/models/neo_unify/modeling_qwen3.py:183-200,
// q/k half norms and t/h/w RoPE :444-468, rotate-half :219-250, SwiGLU :203-217.
#include "host_common.h"
#include "sm100_common.cuh"

namespace snu1 {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int THREADS>
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) t += scratch[i];
  return t;
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

// ---------------------------------------------------------------------------
// RMSNorm over the hidden dimension, gain chosen per 128-row tile.
// ---------------------------------------------------------------------------
constexpr int RN_THREADS = 256;

__global__ void __launch_bounds__(RN_THREADS)
    rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gain,
                       const int* __restrict__ tile_group, __nv_bfloat16* __restrict__ y,
                       float* __restrict__ rstd_out, int rows, int H, float eps) {
  __shared__ float scratch[RN_THREADS / 32];
  const int nvec = H / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    int g = tile_group ? tile_group[row >> 7] : 0;
    if (g < 0) g = 0;
    const uint4* xr = reinterpret_cast<const uint4*>(x + (long long)row * H);
    const uint4* gr = reinterpret_cast<const uint4*>(gain + (long long)g * H);
    uint4* yr = reinterpret_cast<uint4*>(y + (long long)row * H);
    float ss = 0.f;
    for (int v = threadIdx.x; v < nvec; v += RN_THREADS) {
      float f[8];
      unpack8(xr[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    ss = block_sum<RN_THREADS>(ss, scratch);
    const float rstd = rsqrtf(ss / H + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
    for (int v = threadIdx.x; v < nvec; v += RN_THREADS) {
      float f[8], w[8];
      unpack8(xr[v], f);
      unpack8(gr[v], w);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * rstd * w[i];
      yr[v] = pack8(f);
    }
  }
}

// One warp per row, the row held in registers (VPL 16-byte vectors per lane): no block barrier, one read of x,
// VPL independent loads in flight per lane.  Used when H = 256 * VPL; other widths take the kernel above.
template <int VPL>
__global__ void __launch_bounds__(RN_THREADS, 2)
    rmsnorm_fwd_warp_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gain,
                            const int* __restrict__ tile_group, __nv_bfloat16* __restrict__ y,
                            float* __restrict__ rstd_out, int rows, float eps) {
  constexpr int H = 256 * VPL;
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * (RN_THREADS / 32);
  for (int row = blockIdx.x * (RN_THREADS / 32) + (threadIdx.x >> 5); row < rows; row += warps) {
    int g = tile_group ? tile_group[row >> 7] : 0;
    if (g < 0) g = 0;
    const uint4* xr = reinterpret_cast<const uint4*>(x + (long long)row * H);
    const uint4* gr = reinterpret_cast<const uint4*>(gain + (long long)g * H);
    uint4* yr = reinterpret_cast<uint4*>(y + (long long)row * H);
    uint4 v[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) v[j] = xr[lane + 32 * j];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      float f[8];
      unpack8(v[j], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / H + eps);
    if (lane == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      float f[8], w[8];
      unpack8(v[j], f);
      unpack8(__ldg(gr + lane + 32 * j), w);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * rstd * w[i];
      yr[lane + 32 * j] = pack8(f);
    }
  }
}

// dx = rstd * (g*dy - xhat * mean(g*dy*xhat)) (+ dres);  dgain[g] += sum_rows dy * xhat.
// Each CTA owns ROWS_PER_CTA consecutive rows of one tile and keeps its gain
// gradient in registers until the end, then adds it to the fp32 accumulator.
constexpr int RN_ROWS_PER_CTA = 32;
constexpr int RN_MAX_VEC_PER_THREAD = 4;  // H <= 8 * 256 * 4 = 8192

__global__ void __launch_bounds__(RN_THREADS)
    rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                       const __nv_bfloat16* __restrict__ gain, const float* __restrict__ rstd_in,
                       const int* __restrict__ tile_group, const __nv_bfloat16* __restrict__ dres,
                       __nv_bfloat16* __restrict__ dx, float* __restrict__ dgain, int rows, int H) {
  __shared__ float scratch[RN_THREADS / 32];
  const int nvec = H / 8;
  const int row0 = blockIdx.x * RN_ROWS_PER_CTA;
  if (row0 >= rows) return;
  int g = tile_group ? tile_group[row0 >> 7] : 0;
  const bool tile_ok = g >= 0;
  if (g < 0) g = 0;
  const uint4* gr = reinterpret_cast<const uint4*>(gain + (long long)g * H);
  float dg[RN_MAX_VEC_PER_THREAD][8];
#pragma unroll
  for (int j = 0; j < RN_MAX_VEC_PER_THREAD; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) dg[j][i] = 0.f;

  for (int r = 0; r < RN_ROWS_PER_CTA; ++r) {
    const int row = row0 + r;
    if (row >= rows) break;
    const uint4* xr = reinterpret_cast<const uint4*>(x + (long long)row * H);
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + (long long)row * H);
    const float rstd = rstd_in[row];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < RN_MAX_VEC_PER_THREAD; ++j) {
      const int v = threadIdx.x + j * RN_THREADS;
      if (v < nvec) {
        float xf[8], dyf[8], w[8];
        unpack8(xr[v], xf);
        unpack8(dyr[v], dyf);
        unpack8(gr[v], w);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xh = xf[i] * rstd;
          dot += dyf[i] * w[i] * xh;
          dg[j][i] += dyf[i] * xh;
        }
      }
    }
    dot = block_sum<RN_THREADS>(dot, scratch) / H;
    uint4* dxr = reinterpret_cast<uint4*>(dx + (long long)row * H);
    const uint4* drr = dres ? reinterpret_cast<const uint4*>(dres + (long long)row * H) : nullptr;
#pragma unroll
    for (int j = 0; j < RN_MAX_VEC_PER_THREAD; ++j) {
      const int v = threadIdx.x + j * RN_THREADS;
      if (v < nvec) {
        float xf[8], dyf[8], w[8], o[8];
        unpack8(xr[v], xf);
        unpack8(dyr[v], dyf);
        unpack8(gr[v], w);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rstd * (dyf[i] * w[i] - xf[i] * rstd * dot);
        if (drr) {
          float rf[8];
          unpack8(drr[v], rf);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += rf[i];
        }
        dxr[v] = pack8(o);
      }
    }
  }
  if (dgain && tile_ok) {
#pragma unroll
    for (int j = 0; j < RN_MAX_VEC_PER_THREAD; ++j) {
      const int v = threadIdx.x + j * RN_THREADS;
      if (v < nvec) {
#pragma unroll
        for (int i = 0; i < 8; ++i) atomicAdd(dgain + (long long)g * H + v * 8 + i, dg[j][i]);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// q/k half-head RMSNorm + three-axis RoPE.  head_dim is 128: dims [0,64) carry
// the temporal axis, [64,96) the row axis, [96,128) the column axis.  One warp
// handles one head of one token; lane l owns elements [4l, 4l+4).
//   gains: [groups][4][64] = (q_t, q_hw, k_t, k_hw)
//   pos:   [3][rows] int32 (t, h, w)
// ---------------------------------------------------------------------------
constexpr int QK_THREADS = 128;

struct RopeTable {
  float c[64];  // cos for t pairs [0,32), h pairs [32,48), w pairs [48,64)
  float s[64];
};

__device__ __forceinline__ void fill_rope_table(RopeTable* tab, const int* pos, int rows, int row,
                                                const float* inv_t, const float* inv_hw) {
  for (int i = threadIdx.x; i < 64; i += blockDim.x) {
    float ang;
    if (i < 32) ang = (float)pos[row] * inv_t[i];
    else if (i < 48) ang = (float)pos[rows + row] * inv_hw[i - 32];
    else ang = (float)pos[2 * rows + row] * inv_hw[i - 48];
    float sn, cs;
    sincosf(ang, &sn, &cs);
    tab->c[i] = cs;
    tab->s[i] = sn;
  }
}

// lane -> (table base index, partner xor, sign) for its 4 elements
__device__ __forceinline__ void rope_lane_info(int lane, int& tab0, int& pxor, bool& first_half) {
  if (lane < 16) {  // t block, pairs (i, i+32), 8 lanes per half
    pxor = 8;
    first_half = lane < 8;
    tab0 = (lane & 7) * 4;
  } else if (lane < 24) {  // h block, pairs (i, i+16), 4 lanes per half
    pxor = 4;
    first_half = lane < 20;
    tab0 = 32 + (lane & 3) * 4;
  } else {  // w block
    pxor = 4;
    first_half = lane < 28;
    tab0 = 48 + (lane & 3) * 4;
  }
}

__global__ void __launch_bounds__(QK_THREADS)
    qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, long long ld_in,
                           __nv_bfloat16* __restrict__ out, long long ld_out,
                           const __nv_bfloat16* __restrict__ gains,
                           const int* __restrict__ tile_group, const int* __restrict__ pos,
                           const float* __restrict__ inv_t, const float* __restrict__ inv_hw,
                           int rows, int n_q_heads, int n_kv_heads, float eps) {
  __shared__ RopeTable tab;
  const int row = blockIdx.x;
  int g = tile_group ? tile_group[row >> 7] : 0;
  if (g < 0) g = 0;
  fill_rope_table(&tab, pos, rows, row, inv_t, inv_hw);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int tab0, pxor;
  bool first;
  rope_lane_info(lane, tab0, pxor, first);
  const int nheads = n_q_heads + n_kv_heads;
  for (int h = warp; h < nheads; h += QK_THREADS / 32) {
    const bool is_k = h >= n_q_heads;
    const __nv_bfloat16* src = qkv + (long long)row * ld_in + h * 128 + lane * 4;
    const uint2 raw = *reinterpret_cast<const uint2*>(src);
    float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    float v[4] = {a.x, a.y, b.x, b.y};
    float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);  // 16-lane halves
    const float rstd = rsqrtf(ss / 64.f + eps);
    const int which = (is_k ? 2 : 0) + (lane >= 16 ? 1 : 0);
    const __nv_bfloat16* gp = gains + ((long long)g * 4 + which) * 64 + (lane & 15) * 4;
    float n[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) n[i] = v[i] * rstd * __bfloat162float(gp[i]);
    float o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, n[i], pxor);
      const float cs = tab.c[tab0 + i], sn = tab.s[tab0 + i];
      o[i] = first ? (n[i] * cs - other * sn) : (n[i] * cs + other * sn);
    }
    uint2 packed;
    packed.x = pack_bf16x2(o[0], o[1]);
    packed.y = pack_bf16x2(o[2], o[3]);
    *reinterpret_cast<uint2*>(out + (long long)row * ld_out + h * 128 + lane * 4) = packed;
  }
}

// Backward: d_in = d(norm)(R^T d_out); dgains[g][which][64] += sum d_n * xhat.
// `d` is updated in place (ld_d), qkv holds the saved pre-norm projections.
__global__ void __launch_bounds__(QK_THREADS)
    qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ qkv, long long ld_in,
                           __nv_bfloat16* __restrict__ d, long long ld_d,
                           const __nv_bfloat16* __restrict__ gains, float* __restrict__ dgains,
                           const int* __restrict__ tile_group, const int* __restrict__ pos,
                           const float* __restrict__ inv_t, const float* __restrict__ inv_hw,
                           int rows, int rows_per_cta, int n_q_heads, int n_kv_heads, float eps) {
  __shared__ RopeTable tab;
  __shared__ float sdg[4 * 64];
  for (int i = threadIdx.x; i < 256; i += QK_THREADS) sdg[i] = 0.f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int tab0, pxor;
  bool first;
  rope_lane_info(lane, tab0, pxor, first);
  const int nheads = n_q_heads + n_kv_heads;
  const int row_begin = blockIdx.x * rows_per_cta;
  int g = tile_group ? tile_group[row_begin >> 7] : 0;  // rows_per_cta divides 128
  const bool tile_ok = g >= 0;
  if (g < 0) g = 0;
  float acc_q[4] = {0.f, 0.f, 0.f, 0.f};
  float acc_k[4] = {0.f, 0.f, 0.f, 0.f};
  for (int r = 0; r < rows_per_cta; ++r) {
    const int row = row_begin + r;
    if (row >= rows) break;
    __syncthreads();
    fill_rope_table(&tab, pos, rows, row, inv_t, inv_hw);
    __syncthreads();
    for (int h = warp; h < nheads; h += QK_THREADS / 32) {
      const bool is_k = h >= n_q_heads;
      const uint2 raw =
          *reinterpret_cast<const uint2*>(qkv + (long long)row * ld_in + h * 128 + lane * 4);
      float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
      float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
      float v[4] = {a.x, a.y, b.x, b.y};
      float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float rstd = rsqrtf(ss / 64.f + eps);
      __nv_bfloat16* dp = d + (long long)row * ld_d + h * 128 + lane * 4;
      const uint2 draw = *reinterpret_cast<const uint2*>(dp);
      float2 da = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&draw.x));
      float2 db = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&draw.y));
      float dy[4] = {da.x, da.y, db.x, db.y};
      const int which = (is_k ? 2 : 0) + (lane >= 16 ? 1 : 0);
      const __nv_bfloat16* gp = gains + ((long long)g * 4 + which) * 64 + (lane & 15) * 4;
      float dn[4], xh[4], dxh[4];
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, dy[i], pxor);
        const float cs = tab.c[tab0 + i], sn = tab.s[tab0 + i];
        dn[i] = first ? (dy[i] * cs + other * sn) : (dy[i] * cs - other * sn);
        xh[i] = v[i] * rstd;
        dxh[i] = dn[i] * __bfloat162float(gp[i]);
        dot += dxh[i] * xh[i];
        if (is_k) acc_k[i] += dn[i] * xh[i];
        else acc_q[i] += dn[i] * xh[i];
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      dot *= (1.f / 64.f);
      float dx[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) dx[i] = rstd * (dxh[i] - xh[i] * dot);
      uint2 packed;
      packed.x = pack_bf16x2(dx[0], dx[1]);
      packed.y = pack_bf16x2(dx[2], dx[3]);
      *reinterpret_cast<uint2*>(dp) = packed;
    }
  }
  // lane l holds gain-gradient partials for gain (lane>=16 ? hw : t), elements (l&15)*4..+4
  const int half = lane >= 16 ? 1 : 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    atomicAdd(&sdg[(0 + half) * 64 + (lane & 15) * 4 + i], acc_q[i]);
    atomicAdd(&sdg[(2 + half) * 64 + (lane & 15) * 4 + i], acc_k[i]);
  }
  __syncthreads();
  if (dgains && tile_ok)
    for (int i = threadIdx.x; i < 256; i += QK_THREADS) atomicAdd(dgains + (long long)g * 256 + i, sdg[i]);
}

// ---------------------------------------------------------------------------
// SwiGLU on the fused projection [rows][gate(F) | up(F)].
// ---------------------------------------------------------------------------
// rows_dev (optional): the number of rows in use, read on the device, for buffers sized for a worst case
// sigmoid(x) = 0.5 tanh(x / 2) + 0.5 with the hardware tanh: one special-function operation per element (the
// exp + divide form costs two plus a Newton step, which made these kernels instruction-bound, not memory-bound).
__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// One row per CTA step, columns strided over the threads: no 64-bit division per element vector.
__global__ void __launch_bounds__(256)
    swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ act, long long rows, int F,
                      const int* __restrict__ rows_dev) {
  if (rows_dev != nullptr && *rows_dev < rows) rows = *rows_dev;
  const int fv = F / 8;
  const int rpc = fv >= 256 ? 1 : 256 / fv;   // narrow rows (expert FFNs): several rows per CTA step
  const int tr = rpc == 1 ? 0 : threadIdx.x / fv;
  const int tc = threadIdx.x - tr * fv;
  for (long long r0 = (long long)blockIdx.x * rpc; r0 < rows; r0 += (long long)gridDim.x * rpc) {
    const long long r = r0 + tr;
    if (tr >= rpc || r >= rows) continue;
    const uint4* base = reinterpret_cast<const uint4*>(gu + r * 2 * F);
    uint4* out = reinterpret_cast<uint4*>(act + r * F);
#pragma unroll 2
    for (int c = tc; c < fv; c += 256) {
      float gt[8], up[8], o[8];
      unpack8(base[c], gt);
      unpack8(base[fv + c], up);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float h = 0.5f * gt[j];
        o[j] = fmaf(h, fast_tanh(h), h) * up[j];   // silu(g) = g sigmoid(g) = h tanh(h) + h
      }
      out[c] = pack8(o);
    }
  }
}

__global__ void __launch_bounds__(256)
    swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dact,
                      __nv_bfloat16* __restrict__ dgu, long long rows, int F, const int* __restrict__ rows_dev) {
  if (rows_dev != nullptr && *rows_dev < rows) rows = *rows_dev;
  const int fv = F / 8;
  const int rpc = fv >= 256 ? 1 : 256 / fv;
  const int tr = rpc == 1 ? 0 : threadIdx.x / fv;
  const int tc = threadIdx.x - tr * fv;
  for (long long r0 = (long long)blockIdx.x * rpc; r0 < rows; r0 += (long long)gridDim.x * rpc) {
    const long long r = r0 + tr;
    if (tr >= rpc || r >= rows) continue;
    const uint4* base = reinterpret_cast<const uint4*>(gu + r * 2 * F);
    const uint4* dab = reinterpret_cast<const uint4*>(dact + r * F);
    uint4* ob = reinterpret_cast<uint4*>(dgu + r * 2 * F);
#pragma unroll 2
    for (int c = tc; c < fv; c += 256) {
      float gt[8], up[8], da[8], dgt[8], dup[8];
      unpack8(base[c], gt);
      unpack8(base[fv + c], up);
      unpack8(dab[c], da);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float sg = fmaf(0.5f, fast_tanh(0.5f * gt[j]), 0.5f);
        const float silu = gt[j] * sg;
        dup[j] = da[j] * silu;
        dgt[j] = da[j] * up[j] * (sg + silu * (1.f - sg));
      }
      ob[c] = pack8(dgt);
      ob[fv + c] = pack8(dup);
    }
  }
}

}  // namespace snu1

using namespace snu1;

SNU1_API int snu1_rmsnorm_fwd(const void* x, const void* gain, const int* tile_group, void* y,
                              float* rstd, int rows, int H, float eps, void* stream) {
  if (H % 8 != 0 || rows <= 0) {
    set_last_error("rmsnorm_fwd: H must be a multiple of 8 (H=%d rows=%d)", H, rows);
    return kHostBadArg;
  }
  {
    const int wgrid = (rows + 7) / 8 < 148 * 8 ? (rows + 7) / 8 : 148 * 8;
    const __nv_bfloat16 *xp = (const __nv_bfloat16*)x, *gp = (const __nv_bfloat16*)gain;
    __nv_bfloat16* yp = (__nv_bfloat16*)y;
    cudaStream_t st = (cudaStream_t)stream;
    bool done = true;
    switch (H) {
      case 256: rmsnorm_fwd_warp_kernel<1><<<wgrid, RN_THREADS, 0, st>>>(xp, gp, tile_group, yp, rstd, rows, eps); break;
      case 512: rmsnorm_fwd_warp_kernel<2><<<wgrid, RN_THREADS, 0, st>>>(xp, gp, tile_group, yp, rstd, rows, eps); break;
      case 1024: rmsnorm_fwd_warp_kernel<4><<<wgrid, RN_THREADS, 0, st>>>(xp, gp, tile_group, yp, rstd, rows, eps); break;
      case 2048: rmsnorm_fwd_warp_kernel<8><<<wgrid, RN_THREADS, 0, st>>>(xp, gp, tile_group, yp, rstd, rows, eps); break;
      case 4096: rmsnorm_fwd_warp_kernel<16><<<wgrid, RN_THREADS, 0, st>>>(xp, gp, tile_group, yp, rstd, rows, eps); break;
      default: done = false;
    }
    if (done) {
      SNU1_CUDA_CHECK(cudaGetLastError());
      return kHostOk;
    }
  }
  int grid = rows < 148 * 8 ? rows : 148 * 8;
  rmsnorm_fwd_kernel<<<grid, RN_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)gain, tile_group, (__nv_bfloat16*)y, rstd,
      rows, H, eps);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_rmsnorm_bwd(const void* dy, const void* x, const void* gain, const float* rstd,
                              const int* tile_group, const void* dres, void* dx, float* dgain,
                              int rows, int H, void* stream) {
  if (H % 8 != 0 || H > 8 * RN_THREADS * RN_MAX_VEC_PER_THREAD || rows <= 0) {
    set_last_error("rmsnorm_bwd: unsupported H=%d (multiple of 8, at most %d)", H,
                   8 * RN_THREADS * RN_MAX_VEC_PER_THREAD);
    return kHostBadArg;
  }
  int grid = (rows + RN_ROWS_PER_CTA - 1) / RN_ROWS_PER_CTA;
  rmsnorm_bwd_kernel<<<grid, RN_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gain, rstd,
      tile_group, (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, dgain, rows, H);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_qknorm_rope_fwd(const void* qkv, long long ld_in, void* out, long long ld_out,
                                  const void* gains, const int* tile_group, const int* pos,
                                  const float* inv_t, const float* inv_hw, int rows, int n_q_heads,
                                  int n_kv_heads, float eps, void* stream) {
  if (rows <= 0 || ld_in % 4 != 0 || ld_out % 4 != 0) {
    set_last_error("qknorm_rope_fwd: bad rows / strides");
    return kHostBadArg;
  }
  qknorm_rope_fwd_kernel<<<rows, QK_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)qkv, ld_in, (__nv_bfloat16*)out, ld_out, (const __nv_bfloat16*)gains,
      tile_group, pos, inv_t, inv_hw, rows, n_q_heads, n_kv_heads, eps);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_qknorm_rope_bwd(const void* qkv, long long ld_in, void* d, long long ld_d,
                                  const void* gains, float* dgains, const int* tile_group,
                                  const int* pos, const float* inv_t, const float* inv_hw, int rows,
                                  int n_q_heads, int n_kv_heads, float eps, void* stream) {
  if (rows <= 0 || ld_in % 4 != 0 || ld_d % 4 != 0) {
    set_last_error("qknorm_rope_bwd: bad rows / strides");
    return kHostBadArg;
  }
  const int rows_per_cta = 16;
  const int grid = (rows + rows_per_cta - 1) / rows_per_cta;
  qknorm_rope_bwd_kernel<<<grid, QK_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)qkv, ld_in, (__nv_bfloat16*)d, ld_d, (const __nv_bfloat16*)gains,
      dgains, tile_group, pos, inv_t, inv_hw, rows, rows_per_cta, n_q_heads, n_kv_heads, eps);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

// rows_dev may be null; otherwise only min(rows, *rows_dev) rows are processed (count known on the device only)
SNU1_API int snu1_swiglu_fwd_dyn(const void* gu, void* act, long long rows, int F, const int* rows_dev, void* stream) {
  if (F % 8 != 0 || rows <= 0) {
    set_last_error("swiglu_fwd: F must be a multiple of 8");
    return kHostBadArg;
  }
  const int rpc = F / 8 >= 256 ? 1 : 256 / (F / 8);
  const long long steps = (rows + rpc - 1) / rpc;
  int grid = (int)(steps < 148 * 8 ? steps : 148 * 8);
  swiglu_fwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)gu,
                                                            (__nv_bfloat16*)act, rows, F, rows_dev);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_swiglu_fwd(const void* gu, void* act, long long rows, int F, void* stream) {
  return snu1_swiglu_fwd_dyn(gu, act, rows, F, nullptr, stream);
}

SNU1_API int snu1_swiglu_bwd_dyn(const void* gu, const void* dact, void* dgu, long long rows, int F,
                                 const int* rows_dev, void* stream) {
  if (F % 8 != 0 || rows <= 0) {
    set_last_error("swiglu_bwd: F must be a multiple of 8");
    return kHostBadArg;
  }
  const int rpc = F / 8 >= 256 ? 1 : 256 / (F / 8);
  const long long steps = (rows + rpc - 1) / rpc;
  int grid = (int)(steps < 148 * 8 ? steps : 148 * 8);
  swiglu_bwd_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gu, (const __nv_bfloat16*)dact, (__nv_bfloat16*)dgu, rows, F, rows_dev);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_swiglu_bwd(const void* gu, const void* dact, void* dgu, long long rows, int F,
                             void* stream) {
  return snu1_swiglu_bwd_dyn(gu, dact, dgu, rows, F, nullptr, stream);
}
