// Mixture-of-experts routing kernels: fp32 softmax gate with top-k selection and
// renormalisation, deterministic slot assignment into expert segments padded to the
// GEMM tile height, token gather into that layout, weighted combine, and their
// backward passes.  The expert FFNs themselves are the grouped tcgen05 GEMM
// (gemm_sm100.cu, group_mode 1 / 2) running over the padded segments.
//
// Reference: router and dropless dispatch training/sensenovalm/model/moe/dropless_layer_qwen.py:90-163,
// 352-506, 573-660 (host-synchronising split sizes, argsort / index permute, grouped_gemm.ops.permute);
// inference block src/sensenova_u1/models/neo_unify/modeling_qwen3_moe.py:51-119.
// Here split sizes never leave the device.
#include "host_common.h"
#include "sm100_common.cuh"

namespace snu1 {

constexpr int kMaxExperts = 256;
constexpr int kMaxTopK = 16;

// One warp per token.  logits [R,E] fp32 -> probs (optional, fp32 [R,E]), top-k ids / weights.
// Ties are broken towards the lower expert index (as torch.topk on a sorted scan would for
// equal values is unspecified; the oracle test uses distinct values).
__global__ void __launch_bounds__(256)
    moe_router_kernel(const float* __restrict__ logits, int R, int E, int K, int norm_topk,
                      float* __restrict__ probs_out, int* __restrict__ top_idx, float* __restrict__ top_w,
                      int* __restrict__ counts, const int* __restrict__ row_valid,
                      const float* __restrict__ sel_bias, float* __restrict__ lse_out,
                      const int* __restrict__ row_class, int* __restrict__ class_counts) {
  const int row = (blockIdx.x * 256 + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= R) return;
  const bool valid = row_valid == nullptr || row_valid[row] != 0;
  constexpr int PER = kMaxExperts / 32;
  float v[PER];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? logits[(long long)row * E + e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    v[i] = lane + 32 * i < E ? __expf(v[i] - mx) : 0.f;
    sum += v[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float inv = 1.f / sum;
  if (lse_out && lane == 0) lse_out[row] = valid ? mx + __logf(sum) : 0.f;     // log-sum-exp of the row (z-loss)
  // selection score: the probability, plus the per-expert correction bias of bias-based ("aux-free") load
  // balancing when given; the bias steers which experts are picked, the mixing weights stay the probabilities
  float sc[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    v[i] *= inv;
    const int e = lane + 32 * i;
    if (probs_out && e < E) probs_out[(long long)row * E + e] = v[i];
    sc[i] = e < E ? v[i] + (sel_bias ? sel_bias[e] : 0.f) : -INFINITY;
  }
  float wsum = 0.f;
  float my_w = 0.f;
  int my_e = -1;
  for (int k = 0; k < K; ++k) {
    float best = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + 32 * i;
      if (e < E && (sc[i] > best)) {
        best = sc[i];
        be = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) {
        best = ob;
        be = oe;
      }
    }
    const float pw = __shfl_sync(0xffffffffu, v[be >> 5], be & 31);     // the chosen expert's probability
    if ((be & 31) == lane) sc[be >> 5] = -INFINITY;  // remove from further rounds
    if (lane == k) {
      my_w = pw;
      my_e = be;
    }
    wsum += pw;
  }
  if (lane < K) {
    const float w = norm_topk ? my_w / wsum : my_w;
    top_idx[(long long)row * K + lane] = valid ? my_e : -1;
    top_w[(long long)row * K + lane] = valid ? w : 0.f;
    if (valid) {
      atomicAdd(counts + my_e, 1);
      if (class_counts && row_class) atomicAdd(class_counts + row_class[row] * E + my_e, 1);
    }
  }
}

// Single block: exclusive scan of counts padded to 128 -> segment starts; also the per-tile
// expert map for the grouped GEMM and the per-expert row ranges for weight gradients.
__global__ void moe_segments_kernel(const int* __restrict__ counts, int E, int max_tiles,
                                    int* __restrict__ seg_start, int* __restrict__ seg_end,
                                    int* __restrict__ tile_group, int* __restrict__ total_rows) {
  __shared__ int s_start[kMaxExperts + 1];
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) {
      s_start[e] = acc;
      acc += (counts[e] + 127) / 128 * 128;
    }
    s_start[E] = acc;
    *total_rows = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    seg_start[e] = s_start[e];
    seg_end[e] = s_start[e] + (counts[e] + 127) / 128 * 128;  // padded: pad rows are zero
  }
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) {
    const int r0 = t * 128;
    int g = -1;
    if (r0 < s_start[E]) {
      int lo = 0, hi = E - 1;  // last e with s_start[e] <= r0
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (s_start[mid] <= r0) lo = mid;
        else hi = mid - 1;
      }
      g = lo;
    }
    tile_group[t] = g;
  }
}

// Deterministic slot assignment: one block per expert scans the (row, k) pairs in order, 1024 pairs per
// iteration (4 consecutive pairs per thread, warp shuffle scan + one shared-memory scan of the 8 warp totals).
__global__ void __launch_bounds__(256)
    moe_assign_kernel(const int* __restrict__ top_idx, int RK, const int* __restrict__ seg_start,
                      int* __restrict__ dest) {
  __shared__ int s_base;
  __shared__ int s_warp[8];
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) s_base = seg_start[e];
  __syncthreads();
  for (int i0 = 0; i0 < RK; i0 += 1024) {
    const int i = i0 + threadIdx.x * 4;
    int idx[4];
    if (i + 3 < RK) {
      const int4 v = *reinterpret_cast<const int4*>(top_idx + i);   // RK * 4 B rows are 16-byte aligned (i % 4 == 0)
      idx[0] = v.x; idx[1] = v.y; idx[2] = v.z; idx[3] = v.w;
    } else {
#pragma unroll
      for (int u = 0; u < 4; ++u) idx[u] = i + u < RK ? top_idx[i + u] : -1;
    }
    int hit[4], c = 0;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      hit[u] = idx[u] == e;
      c += hit[u];
    }
    int incl = c;                                   // inclusive scan of the per-thread counts inside the warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    int before = incl - c, total = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      if (w < warp) before += s_warp[w];
      total += s_warp[w];
    }
    int slot = s_base + before;
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (hit[u]) dest[i + u] = slot++;
    __syncthreads();
    if (threadIdx.x == 0) s_base += total;
    __syncthreads();
  }
}

// xp[dest[row,k]] = x[row]; rows of xp that nobody writes must be zero (caller clears xp).
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ dest,
                                  const int* __restrict__ top_idx, __nv_bfloat16* __restrict__ xp, int R, int K,
                                  int H) {
  const int hv = H / 8;
  const long long total = (long long)R * K * hv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long rk = i / hv;
    const int c = (int)(i - rk * hv);
    if (top_idx[rk] < 0) continue;
    const long long row = rk / K;
    reinterpret_cast<uint4*>(xp + (long long)dest[rk] * H)[c] = reinterpret_cast<const uint4*>(x + row * H)[c];
  }
}

// y[row] = sum_k w[row,k] * yp[dest[row,k]]   (optionally + residual)
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ yp, const int* __restrict__ dest,
                                   const int* __restrict__ top_idx, const float* __restrict__ top_w,
                                   const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ y,
                                   int R, int K, int H) {
  const int hv = H / 8;
  const long long total = (long long)R * hv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / hv;
    const int c = (int)(i - row * hv);
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    if (residual) {
      const uint4 u = reinterpret_cast<const uint4*>(residual + row * H)[c];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] = f.x;
        acc[2 * e + 1] = f.y;
      }
    }
    for (int k = 0; k < K; ++k) {
      const long long rk = row * K + k;
      if (top_idx[rk] < 0) continue;
      const float w = top_w[rk];
      const uint4 u = reinterpret_cast<const uint4*>(yp + (long long)dest[rk] * H)[c];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] += w * f.x;
        acc[2 * e + 1] += w * f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(y + row * H)[c] = o;
  }
}

// backward of combine: dyp[dest] = w * dy[row];  dw[row,k] = <dy[row], yp[dest]>.  One warp per (row,k).
__global__ void __launch_bounds__(256)
    moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ yp,
                           const int* __restrict__ dest, const int* __restrict__ top_idx,
                           const float* __restrict__ top_w, __nv_bfloat16* __restrict__ dyp,
                           float* __restrict__ dw, int R, int K, int H) {
  const long long rk = (blockIdx.x * 256ll + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (rk >= (long long)R * K) return;
  if (top_idx[rk] < 0) {
    if (lane == 0) dw[rk] = 0.f;
    return;
  }
  const long long row = rk / K;
  const float w = top_w[rk];
  const long long d = dest[rk];
  float dot = 0.f;
  for (int c = lane; c < H / 8; c += 32) {
    const uint4 a = reinterpret_cast<const uint4*>(dy + row * H)[c];
    const uint4 b = reinterpret_cast<const uint4*>(yp + d * H)[c];
    const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
    uint4 o;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 fa = __bfloat1622float2(ha[e]), fb = __bfloat1622float2(hb[e]);
      dot += fa.x * fb.x + fa.y * fb.y;
      op[e] = pack_bf16x2(fa.x * w, fa.y * w);
    }
    reinterpret_cast<uint4*>(dyp + d * H)[c] = o;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  if (lane == 0) dw[rk] = dot;
}

// backward of gather: dx[row] (+)= sum_k dxp[dest[row,k]]
__global__ void moe_gather_bwd_kernel(const __nv_bfloat16* __restrict__ dxp, const int* __restrict__ dest,
                                      const int* __restrict__ top_idx, __nv_bfloat16* __restrict__ dx,
                                      int accumulate, int R, int K, int H) {
  const int hv = H / 8;
  const long long total = (long long)R * hv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / hv;
    const int c = (int)(i - row * hv);
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    if (accumulate) {
      const uint4 u = reinterpret_cast<const uint4*>(dx + row * H)[c];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] = f.x;
        acc[2 * e + 1] = f.y;
      }
    }
    for (int k = 0; k < K; ++k) {
      const long long rk = row * K + k;
      if (top_idx[rk] < 0) continue;
      const uint4 u = reinterpret_cast<const uint4*>(dxp + (long long)dest[rk] * H)[c];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] += f.x;
        acc[2 * e + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(dx + row * H)[c] = o;
  }
}

// Router backward.  Inputs: probs [R,E], top ids / normalised weights, dw [R,K] (gradient of the
// normalised weights), plus the load-balancing term  aux_coef * E * f_e / R_valid  on every prob
// (f = routed fraction, treated as constant).  Output: dlogits [R,E] (bf16, for the gate GEMMs).
__global__ void __launch_bounds__(256)
    moe_router_bwd_kernel(const float* __restrict__ probs, const int* __restrict__ top_idx,
                          const float* __restrict__ top_w, const float* __restrict__ dw,
                          const int* __restrict__ counts, float aux_scale, int norm_topk,
                          __nv_bfloat16* __restrict__ dlogits, int R, int E, int K,
                          const int* __restrict__ row_class, const int* __restrict__ class_counts,
                          float aux_scale_c0, float aux_scale_c1, const float* __restrict__ lse, float z_scale) {
  const int row = (blockIdx.x * 256 + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= R) return;
  constexpr int PER = kMaxExperts / 32;
  float p[PER], dp[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    p[i] = e < E ? probs[(long long)row * E + e] : 0.f;
    if (row_class && class_counts) {
      // balance loss per token class (text / image): this row's class term only
      const int c = row_class[row];
      dp[i] = e < E ? (c ? aux_scale_c1 : aux_scale_c0) * (float)class_counts[c * E + e] : 0.f;
    } else {
      dp[i] = e < E ? aux_scale * (float)counts[e] : 0.f;
    }
  }
  const bool valid = top_idx[(long long)row * K] >= 0;
  if (valid) {
    // normalised weight w_k = p_k / S (S = sum of selected probs): dp_k += (dw_k - sum_j dw_j w_j) / S
    float S = 0.f, dot = 0.f;
    for (int k = 0; k < K; ++k) {
      const int e = top_idx[(long long)row * K + k];
      const float pe = __shfl_sync(0xffffffffu, p[e >> 5], e & 31);
      S += pe;
      dot += dw[(long long)row * K + k] * top_w[(long long)row * K + k];
    }
    for (int k = 0; k < K; ++k) {
      const int e = top_idx[(long long)row * K + k];
      const float g = norm_topk ? (dw[(long long)row * K + k] - dot) / S : dw[(long long)row * K + k];
      if ((e & 31) == lane) dp[e >> 5] += g;
    }
  } else {
#pragma unroll
    for (int i = 0; i < PER; ++i) dp[i] = 0.f;
  }
  // softmax backward: dlogit_e = p_e (dp_e - sum_j p_j dp_j)
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) s += p[i] * dp[i];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
#pragma unroll
  // z-loss: z_scale * lse^2 summed over valid rows; d lse / d logit_e = p_e
  const float zg = (lse && valid) ? 2.f * z_scale * lse[row] : 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    if (e < E) dlogits[(long long)row * E + e] = __float2bfloat16_rn(p[i] * (dp[i] - s) + zg * p[i]);
  }
}

static int grid_1d(long long total, int block) {
  long long b = (total + block - 1) / block;
  const long long cap = 148ll * 16;
  return (int)(b < 1 ? 1 : (b < cap ? b : cap));
}

}  // namespace snu1

using namespace snu1;

// counts [E] must be zero on entry.  max_tiles = number of 128-row tiles of the permuted buffer.
static int moe_route_impl(const float* logits, int R, int E, int K, int norm_topk, float* probs,
                          int* top_idx, float* top_w, int* counts, const int* row_valid, int max_tiles,
                          int* seg_start, int* seg_end, int* tile_group, int* total_rows, int* dest,
                          const float* sel_bias, float* lse_out, const int* row_class, int* class_counts,
                          void* stream);

SNU1_API int snu1_moe_route(const float* logits, int R, int E, int K, int norm_topk, float* probs,
                            int* top_idx, float* top_w, int* counts, const int* row_valid, int max_tiles,
                            int* seg_start, int* seg_end, int* tile_group, int* total_rows, int* dest,
                            void* stream) {
  return moe_route_impl(logits, R, E, K, norm_topk, probs, top_idx, top_w, counts, row_valid, max_tiles, seg_start,
                        seg_end, tile_group, total_rows, dest, nullptr, nullptr, nullptr, nullptr, stream);
}

// Routing with the training extras: sel_bias [E] (bias-based balancing: added to the selection score only),
// lse_out [R] (row log-sum-exp for the z-loss), row_class [R] in {0,1} with class_counts [2,E] (zero on entry:
// routed slots per token class, for the class-weighted balance loss).  Any of them may be null.
SNU1_API int snu1_moe_route_ex(const float* logits, int R, int E, int K, int norm_topk, float* probs,
                               int* top_idx, float* top_w, int* counts, const int* row_valid, int max_tiles,
                               int* seg_start, int* seg_end, int* tile_group, int* total_rows, int* dest,
                               const float* sel_bias, float* lse_out, const int* row_class, int* class_counts,
                               void* stream) {
  return moe_route_impl(logits, R, E, K, norm_topk, probs, top_idx, top_w, counts, row_valid, max_tiles, seg_start,
                        seg_end, tile_group, total_rows, dest, sel_bias, lse_out, row_class, class_counts, stream);
}

static int moe_route_impl(const float* logits, int R, int E, int K, int norm_topk, float* probs,
                          int* top_idx, float* top_w, int* counts, const int* row_valid, int max_tiles,
                          int* seg_start, int* seg_end, int* tile_group, int* total_rows, int* dest,
                          const float* sel_bias, float* lse_out, const int* row_class, int* class_counts,
                          void* stream) {
  if (E > kMaxExperts || K > kMaxTopK || K > E || R <= 0) {
    set_last_error("moe_route: unsupported E=%d K=%d (max %d / %d)", E, K, kMaxExperts, kMaxTopK);
    return kHostBadArg;
  }
  cudaStream_t st = (cudaStream_t)stream;
  moe_router_kernel<<<(R * 32 + 255) / 256, 256, 0, st>>>(logits, R, E, K, norm_topk, probs, top_idx, top_w,
                                                          counts, row_valid, sel_bias, lse_out, row_class,
                                                          class_counts);
  if (max_tiles > 0) {   // max_tiles == 0: routing only (the expert-parallel plan lays the tokens out)
    moe_segments_kernel<<<1, 256, 0, st>>>(counts, E, max_tiles, seg_start, seg_end, tile_group, total_rows);
    moe_assign_kernel<<<E, 256, 0, st>>>(top_idx, R * K, seg_start, dest);
  }
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_moe_gather(const void* x, const int* dest, const int* top_idx, void* xp, int R, int K, int H,
                             void* stream) {
  if (H % 8) {
    set_last_error("moe_gather: H must be a multiple of 8");
    return kHostBadArg;
  }
  moe_gather_kernel<<<grid_1d((long long)R * K * (H / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, dest, top_idx, (__nv_bfloat16*)xp, R, K, H);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_moe_combine(const void* yp, const int* dest, const int* top_idx, const float* top_w,
                              const void* residual, void* y, int R, int K, int H, void* stream) {
  if (H % 8) {
    set_last_error("moe_combine: H must be a multiple of 8");
    return kHostBadArg;
  }
  moe_combine_kernel<<<grid_1d((long long)R * (H / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)yp, dest, top_idx, top_w, (const __nv_bfloat16*)residual, (__nv_bfloat16*)y, R, K, H);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_moe_combine_bwd(const void* dy, const void* yp, const int* dest, const int* top_idx,
                                  const float* top_w, void* dyp, float* dw, int R, int K, int H, void* stream) {
  if (H % 8) {
    set_last_error("moe_combine_bwd: H must be a multiple of 8");
    return kHostBadArg;
  }
  const long long warps = (long long)R * K;
  moe_combine_bwd_kernel<<<(int)((warps * 32 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)yp, dest, top_idx, top_w, (__nv_bfloat16*)dyp, dw, R, K, H);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_moe_gather_bwd(const void* dxp, const int* dest, const int* top_idx, void* dx, int accumulate,
                                 int R, int K, int H, void* stream) {
  if (H % 8) {
    set_last_error("moe_gather_bwd: H must be a multiple of 8");
    return kHostBadArg;
  }
  moe_gather_bwd_kernel<<<grid_1d((long long)R * (H / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dxp, dest, top_idx, (__nv_bfloat16*)dx, accumulate, R, K, H);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_moe_router_bwd(const float* probs, const int* top_idx, const float* top_w, const float* dw,
                                 const int* counts, float aux_scale, int norm_topk, void* dlogits, int R, int E,
                                 int K, void* stream) {
  if (E > kMaxExperts || K > kMaxTopK) {
    set_last_error("moe_router_bwd: unsupported E=%d K=%d", E, K);
    return kHostBadArg;
  }
  moe_router_bwd_kernel<<<(R * 32 + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
      probs, top_idx, top_w, dw, counts, aux_scale, norm_topk, (__nv_bfloat16*)dlogits, R, E, K, nullptr, nullptr,
      0.f, 0.f, nullptr, 0.f);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

// Router backward with the class-weighted balance term (row_class / class_counts [2,E] / one scale per class)
// and the z-loss term (lse [R], z_scale = coefficient / valid rows).  Null pointers switch a term off.
SNU1_API int snu1_moe_router_bwd_ex(const float* probs, const int* top_idx, const float* top_w, const float* dw,
                                    const int* counts, float aux_scale, int norm_topk, void* dlogits, int R, int E,
                                    int K, const int* row_class, const int* class_counts, float aux_scale_c0,
                                    float aux_scale_c1, const float* lse, float z_scale, void* stream) {
  if (E > kMaxExperts || K > kMaxTopK) {
    set_last_error("moe_router_bwd: unsupported E=%d K=%d", E, K);
    return kHostBadArg;
  }
  moe_router_bwd_kernel<<<(R * 32 + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
      probs, top_idx, top_w, dw, counts, aux_scale, norm_topk, (__nv_bfloat16*)dlogits, R, E, K, row_class,
      class_counts, aux_scale_c0, aux_scale_c1, lse, z_scale);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

// ===========================================================================
// Expert parallelism over NVLink peer memory: dispatch and combine are peer stores / loads issued by
// the gather / combine kernels themselves; no all-to-all collective and no host-visible split sizes
// (reference: all_to_all_single with host-synchronised split sizes,
// training/sensenovalm/model/moe/dropless_layer_qwen.py:407-506, 662-773; moe/utils.py:15-80).
//
// Layout: rank r owns experts [r * E_loc, (r + 1) * E_loc).  Its permuted buffer holds, per local expert,
// the rows of source rank 0, then 1, ... ; each expert segment is padded to 128 rows.  Every rank derives
// the same layout from the [world][E] count table that the ranks write into each other's memory.
// ===========================================================================
namespace snu1 {

struct EpPeers {
  void* p[8];
};

// counts_all on every rank: [world][E]; each rank stores its own row into all peers.
__global__ void moe_ep_put_counts_kernel(const int* __restrict__ counts, EpPeers counts_all, int world, int my_rank,
                                         int E) {
  for (int i = threadIdx.x; i < world * E; i += blockDim.x) {
    const int r = i / E, e = i - r * E;
    reinterpret_cast<int*>(counts_all.p[r])[my_rank * E + e] = counts[e];
  }
}

// From counts_all: base[e] = first row (in the owner's buffer) of MY tokens for global expert e;
// seg_start / seg_end / tile_group / total_rows of MY local experts.
__global__ void moe_ep_plan_kernel(const int* __restrict__ counts_all, int world, int my_rank, int E, int E_loc,
                                   int max_tiles, int* __restrict__ base, int* __restrict__ seg_start,
                                   int* __restrict__ seg_end, int* __restrict__ seg_fill,
                                   int* __restrict__ tile_group, int* __restrict__ total_rows, int* status) {
  __shared__ int s_start[kMaxExperts + 1];
  __shared__ int s_tot[kMaxExperts], s_before[kMaxExperts];
  // per expert, in parallel: rows from all ranks, and rows from the ranks before mine
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int tot = 0, before = 0;
    for (int src = 0; src < world; ++src) {
      const int c = counts_all[src * E + e];
      if (src < my_rank) before += c;
      tot += c;
    }
    s_tot[e] = tot;
    s_before[e] = before;
  }
  __syncthreads();
  // per owner, one thread: running offset over its (few) local experts
  if (threadIdx.x < world) {
    const int owner = threadIdx.x;
    const int lim = max_tiles * 128;
    int acc = 0;
    for (int j = 0; j < E_loc; ++j) {
      const int e = owner * E_loc + j;
      const int tot = s_tot[e];
      base[e] = acc + s_before[e];
      if (owner == my_rank) {
        // clamped to the receive buffer: on overflow (reported below) the segments past the end are empty
        s_start[j] = acc < lim ? acc : lim;
        seg_start[j] = s_start[j];
        seg_end[j] = min(acc + (tot + 127) / 128 * 128, lim);
        seg_fill[j] = min(acc + tot, lim);          // first padding row of the segment
      }
      acc += (tot + 127) / 128 * 128;
    }
    if (owner == my_rank) {
      s_start[E_loc] = acc < lim ? acc : lim;
      *total_rows = s_start[E_loc];
    }
    // a rank whose experts attract more rows than its receive buffer holds: report, never overrun
    if (acc > lim) report_status(status, kBadShape, 8);
  }
  __syncthreads();
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) {
    const int r0 = t * 128;
    int g = -1;
    if (r0 < s_start[E_loc]) {
      int lo = 0, hi = E_loc - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (s_start[mid] <= r0) lo = mid;
        else hi = mid - 1;
      }
      g = lo;
    }
    tile_group[t] = g;
  }
}

// Clears the padding rows (at most 127 per local expert) of two receive buffers: nobody writes them, and
// the weight-gradient GEMMs read whole padded segments.  Replaces clearing the whole worst-case buffer.
__global__ void __launch_bounds__(256)
    moe_ep_zero_pads_kernel(__nv_bfloat16* __restrict__ a, __nv_bfloat16* __restrict__ b,
                            const int* __restrict__ seg_fill, const int* __restrict__ seg_end, int H, int max_rows) {
  const int j = blockIdx.x;
  int r0 = seg_fill[j], r1 = seg_end[j];
  if (r1 > max_rows) r1 = max_rows;
  const int hv = H / 8;
  const uint4 z = make_uint4(0, 0, 0, 0);
  for (long long i = (long long)r0 * hv + threadIdx.x; i < (long long)r1 * hv; i += 256) {
    reinterpret_cast<uint4*>(a)[i] = z;
    if (b != nullptr) reinterpret_cast<uint4*>(b)[i] = z;
  }
}

// dispatch: xp_owner[dest[row,k]] = x[row], a peer store per token copy
__global__ void moe_ep_dispatch_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ dest,
                                       const int* __restrict__ top_idx, EpPeers xp, int E_loc, int R, int K, int H,
                                       int max_rows) {
  const int hv = H / 8;
  const long long total = (long long)R * K * hv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long rk = i / hv;
    const int c = (int)(i - rk * hv);
    const int e = top_idx[rk];
    if (e < 0 || dest[rk] >= max_rows) continue;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(xp.p[e / E_loc]);
    reinterpret_cast<uint4*>(dst + (long long)dest[rk] * H)[c] = reinterpret_cast<const uint4*>(x + (rk / K) * H)[c];
  }
}

// combine: y[row] = residual + sum_k w * yp_owner[dest] (peer loads)
__global__ void moe_ep_combine_kernel(EpPeers yp, const int* __restrict__ dest, const int* __restrict__ top_idx,
                                      const float* __restrict__ top_w, const __nv_bfloat16* __restrict__ residual,
                                      __nv_bfloat16* __restrict__ y, int E_loc, int R, int K, int H, int max_rows) {
  const int hv = H / 8;
  const long long total = (long long)R * hv;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / hv;
    const int c = (int)(i - row * hv);
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    if (residual) {
      const uint4 u = reinterpret_cast<const uint4*>(residual + row * H)[c];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] = f.x;
        acc[2 * e + 1] = f.y;
      }
    }
    for (int k = 0; k < K; ++k) {
      const long long rk = row * K + k;
      const int ex = top_idx[rk];
      // a copy that did not fit the owner's receive buffer was never dispatched (the plan kernel has
      // already reported the overflow): it contributes nothing instead of reading out of bounds
      if (ex < 0 || dest[rk] >= max_rows) continue;
      const float w = top_w ? top_w[rk] : 1.f;
      const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(yp.p[ex / E_loc]);
      const uint4 u = reinterpret_cast<const uint4*>(src + (long long)dest[rk] * H)[c];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] += w * f.x;
        acc[2 * e + 1] += w * f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(y + row * H)[c] = o;
  }
}

// backward of combine across ranks: dyp_owner[dest] = w * dy[row] (peer store); dw = <dy[row], yp_owner[dest]>
__global__ void __launch_bounds__(256)
    moe_ep_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dy, EpPeers yp, EpPeers dyp,
                              const int* __restrict__ dest, const int* __restrict__ top_idx,
                              const float* __restrict__ top_w, float* __restrict__ dw, int E_loc, int R, int K,
                              int H, int max_rows) {
  const long long rk = (blockIdx.x * 256ll + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (rk >= (long long)R * K) return;
  const int ex = top_idx[rk];
  if (ex < 0 || dest[rk] >= max_rows) {
    if (lane == 0) dw[rk] = 0.f;
    return;
  }
  const long long row = rk / K;
  const float w = top_w[rk];
  const long long d = dest[rk];
  const __nv_bfloat16* ysrc = reinterpret_cast<const __nv_bfloat16*>(yp.p[ex / E_loc]);
  __nv_bfloat16* ddst = reinterpret_cast<__nv_bfloat16*>(dyp.p[ex / E_loc]);
  float dot = 0.f;
  for (int c = lane; c < H / 8; c += 32) {
    const uint4 a = reinterpret_cast<const uint4*>(dy + row * H)[c];
    const uint4 b = reinterpret_cast<const uint4*>(ysrc + d * H)[c];
    const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
    uint4 o;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 fa = __bfloat1622float2(ha[e]), fb = __bfloat1622float2(hb[e]);
      dot += fa.x * fb.x + fa.y * fb.y;
      op[e] = pack_bf16x2(fa.x * w, fa.y * w);
    }
    reinterpret_cast<uint4*>(ddst + d * H)[c] = o;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  if (lane == 0) dw[rk] = dot;
}

static int fill_ep(EpPeers* out, const long long* ptrs, int world) {
  if (world < 1 || world > 8) {
    set_last_error("expert-parallel kernels support 1..8 ranks (got %d)", world);
    return kHostBadArg;
  }
  for (int i = 0; i < 8; ++i) out->p[i] = i < world ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return kHostOk;
}

}  // namespace snu1

SNU1_API int snu1_moe_ep_put_counts(const int* counts, const long long* counts_all_ptrs, int world, int my_rank,
                                    int E, void* stream) {
  EpPeers p;
  int rc = fill_ep(&p, counts_all_ptrs, world);
  if (rc != kHostOk) return rc;
  moe_ep_put_counts_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(counts, p, world, my_rank, E);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

// After the counts of every rank have arrived: plan + deterministic slot assignment (dest = row in the owner's buffer).
SNU1_API int snu1_moe_ep_plan(const int* counts_all, int world, int my_rank, int E, int max_tiles, int* base,
                              int* seg_start, int* seg_end, int* seg_fill, int* tile_group, int* total_rows,
                              const int* top_idx, int RK, int* dest, void* stream) {
  if (E > kMaxExperts || E % world) {
    set_last_error("moe_ep_plan: E=%d must be a multiple of the expert-parallel size %d and <= %d", E, world,
                   kMaxExperts);
    return kHostBadArg;
  }
  cudaStream_t st = (cudaStream_t)stream;
  moe_ep_plan_kernel<<<1, 256, 0, st>>>(counts_all, world, my_rank, E, E / world, max_tiles, base, seg_start, seg_end,
                                        seg_fill, tile_group, total_rows, device_status_word());
  moe_assign_kernel<<<E, 256, 0, st>>>(top_idx, RK, base, dest);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_moe_ep_dispatch(const void* x, const int* dest, const int* top_idx, const long long* xp_ptrs,
                                  int world, int E_loc, int R, int K, int H, int max_rows, void* stream) {
  EpPeers p;
  int rc = fill_ep(&p, xp_ptrs, world);
  if (rc != kHostOk) return rc;
  moe_ep_dispatch_kernel<<<grid_1d((long long)R * K * (H / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, dest, top_idx, p, E_loc, R, K, H, max_rows);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

// Clears the padding rows of receive buffers a and b (b may be null); see moe_ep_zero_pads_kernel.
SNU1_API int snu1_moe_ep_zero_pads(void* a, void* b, const int* seg_fill, const int* seg_end, int E_loc, int H,
                                   int max_rows, void* stream) {
  if (H % 8 || E_loc <= 0) {
    set_last_error("moe_ep_zero_pads: bad sizes E_loc=%d H=%d", E_loc, H);
    return kHostBadArg;
  }
  moe_ep_zero_pads_kernel<<<E_loc, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)a, (__nv_bfloat16*)b, seg_fill,
                                                                   seg_end, H, max_rows);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_moe_ep_combine(const long long* yp_ptrs, int world, const int* dest, const int* top_idx,
                                 const float* top_w, const void* residual, void* y, int E_loc, int R, int K, int H,
                                 int max_rows, void* stream) {
  EpPeers p;
  int rc = fill_ep(&p, yp_ptrs, world);
  if (rc != kHostOk) return rc;
  moe_ep_combine_kernel<<<grid_1d((long long)R * (H / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      p, dest, top_idx, top_w, (const __nv_bfloat16*)residual, (__nv_bfloat16*)y, E_loc, R, K, H, max_rows);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_moe_ep_combine_bwd(const void* dy, const long long* yp_ptrs, const long long* dyp_ptrs, int world,
                                     const int* dest, const int* top_idx, const float* top_w, float* dw, int E_loc,
                                     int R, int K, int H, int max_rows, void* stream) {
  EpPeers a, b;
  int rc = fill_ep(&a, yp_ptrs, world);
  if (rc != kHostOk) return rc;
  if ((rc = fill_ep(&b, dyp_ptrs, world)) != kHostOk) return rc;
  const long long warps = (long long)R * K;
  moe_ep_combine_bwd_kernel<<<(int)((warps * 32 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, a, b, dest, top_idx, top_w, dw, E_loc, R, K, H, max_rows);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}
