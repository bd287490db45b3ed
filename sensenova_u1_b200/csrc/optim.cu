// Optimizer-side kernels over flat parameter ranges: squared L2 norm, fused
// unscale + clip + AdamW on an fp32 master that is stored as the bf16 weight
// plus a 16-bit remainder, and the EMA shadow update.
//
// The master weight of element i is the fp32 number whose bit pattern is
// (bits(bf16 weight) << 16) + remainder, with the bf16 weight the
// round-to-nearest of the master.  The model therefore reads correctly rounded
// bf16 weights from the same memory the optimizer updates, and no separate
// fp32 copy or fp32->bf16 cast pass exists
// (reference: training/sensenovalm/solver/optimizer/hybrid_zero_optim.py:891-1031
// keeps a flat fp32 partition and copies it back, :1015-1021).
//
// Gradient clipping needs no host round trip: the kernels read the squared
// global norm from device memory and derive the clip coefficient themselves; a
// non-finite norm makes the step a no-op and raises the `skipped` flag
// (reference: solver/optimizer/utils.py:273-383, hybrid_zero_optim.py:895-930).
#include "host_common.h"
#include "sm100_common.cuh"

namespace snu1 {

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float master_load(__nv_bfloat16 hi, short lo) {
  const uint32_t bits = (static_cast<uint32_t>(__bfloat16_as_ushort(hi)) << 16) + static_cast<int32_t>(lo);
  return __uint_as_float(bits);
}
// Rounds to nearest with ties away from zero (on the bit pattern), so that the
// remainder always fits a signed 16-bit integer: [-0x8000, 0x7fff].
__device__ __forceinline__ void master_store(float w, __nv_bfloat16& hi, short& lo) {
  const uint32_t bits = __float_as_uint(w);
  const uint32_t hb = (bits + 0x8000u) >> 16;
  hi = __ushort_as_bfloat16(static_cast<unsigned short>(hb));
  lo = static_cast<short>(static_cast<int32_t>(bits - (hb << 16)));
}

// 8 consecutive elements of a bf16 / fp32 array as floats (16-byte vector accesses)
template <typename T>
struct Vec8;
template <>
struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = __bfloat1622float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[8]) {
    uint4 u;
    u.x = pack_bf16x2(f[0], f[1]);
    u.y = pack_bf16x2(f[2], f[3]);
    u.z = pack_bf16x2(f[4], f[5]);
    u.w = pack_bf16x2(f[6], f[7]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};
template <>
struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&f)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&f)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
};

template <typename GT>
__global__ void __launch_bounds__(256)
    sumsq_kernel(const GT* __restrict__ g, long long n, float* __restrict__ out) {
  __shared__ float scratch[8];
  float acc = 0.f;
  // 16-byte vector loads over the aligned body (arena ranges are 16-byte aligned), scalar tail
  const bool aligned = (reinterpret_cast<uintptr_t>(g) & 15) == 0;
  const long long nvec = aligned ? (n >> 3) : 0;
  for (long long iv = blockIdx.x * 256ll + threadIdx.x; iv < nvec; iv += (long long)gridDim.x * 256) {
    float f[8];
    Vec8<GT>::load(g + (iv << 3), f);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc += f[e] * f[e];
  }
  for (long long i = (nvec << 3) + blockIdx.x * 256ll + threadIdx.x; i < n; i += (long long)gridDim.x * 256) {
    const float v = to_f<GT>(g[i]);
    acc += v * v;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += scratch[i];
    atomicAdd(out, t);
  }
}

struct AdamArgs {
  long long n;
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;
  float grad_prescale;    // e.g. 1 / (grad accumulation * data-parallel size)
  const float* norm_sq;   // squared norm of the *prescaled-free* gradients, may be null
  float max_norm;         // <= 0: no clipping
  int* skipped;           // set to 1 when the norm is not finite
};

// n must be a multiple of 8 and every pointer 16-byte aligned (arena ranges are).
template <typename GT, typename MT>
__global__ void __launch_bounds__(256)
    adamw_kernel(__nv_bfloat16* __restrict__ p_hi, short* __restrict__ p_lo, const GT* __restrict__ g,
                 MT* __restrict__ m, MT* __restrict__ v, const AdamArgs a) {
  float gscale = a.grad_prescale;
  if (a.norm_sq != nullptr) {
    const float nsq = *a.norm_sq;
    if (!(nsq == nsq) || nsq > 3.0e38f) {  // NaN or inf: skip the step
      if (blockIdx.x == 0 && threadIdx.x == 0 && a.skipped) *a.skipped = 1;
      return;
    }
    if (a.max_norm > 0.f) {
      const float norm = sqrtf(nsq) * a.grad_prescale;
      const float coef = a.max_norm / (norm + 1e-6f);
      if (coef < 1.f) gscale *= coef;
    }
  }
  const float step = a.lr / a.bc1;
  const float inv_sqrt_bc2 = rsqrtf(a.bc2);
  const float decay = 1.f - a.lr * a.weight_decay;
  const long long nvec = a.n >> 3;
  for (long long iv = blockIdx.x * 256ll + threadIdx.x; iv < nvec; iv += (long long)gridDim.x * 256) {
    const long long i = iv << 3;
    float gr[8], mi[8], vi[8];
    Vec8<GT>::load(g + i, gr);
    Vec8<MT>::load(m + i, mi);
    Vec8<MT>::load(v + i, vi);
    const uint4 hu = *reinterpret_cast<const uint4*>(p_hi + i);
    const uint4 lu = *reinterpret_cast<const uint4*>(p_lo + i);
    const unsigned short* hs = reinterpret_cast<const unsigned short*>(&hu);
    const short* ls = reinterpret_cast<const short*>(&lu);
    uint4 ho, lo4;
    unsigned short* hos = reinterpret_cast<unsigned short*>(&ho);
    short* los = reinterpret_cast<short*>(&lo4);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float grad = gr[e] * gscale;
      float w = master_load(__ushort_as_bfloat16(hs[e]), ls[e]);
      mi[e] = a.beta1 * mi[e] + (1.f - a.beta1) * grad;
      vi[e] = a.beta2 * vi[e] + (1.f - a.beta2) * grad * grad;
      const float denom = sqrtf(vi[e]) * inv_sqrt_bc2 + a.eps;
      w = w * decay - step * (mi[e] / denom);
      __nv_bfloat16 hi;
      short lo;
      master_store(w, hi, lo);
      hos[e] = __bfloat16_as_ushort(hi);
      los[e] = lo;
    }
    *reinterpret_cast<uint4*>(p_hi + i) = ho;
    *reinterpret_cast<uint4*>(p_lo + i) = lo4;
    Vec8<MT>::store(m + i, mi);
    Vec8<MT>::store(v + i, vi);
  }
}

__global__ void ema_kernel(float* __restrict__ ema, const __nv_bfloat16* __restrict__ p_hi,
                           const short* __restrict__ p_lo, long long n, float decay) {
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n; i += (long long)gridDim.x * 256) {
    const float w = p_lo ? master_load(p_hi[i], p_lo[i]) : __bfloat162float(p_hi[i]);
    ema[i] = ema[i] * decay + w * (1.f - decay);
  }
}

// out = alpha * x (+ beta * out), element types chosen by flags; used for grad
// casts and for (un)packing fp32 masters into the bf16 + remainder pair.
__global__ void split_master_kernel(const float* __restrict__ w, __nv_bfloat16* __restrict__ hi,
                                    short* __restrict__ lo, long long n) {
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n; i += (long long)gridDim.x * 256) {
    __nv_bfloat16 h;
    short l;
    master_store(w[i], h, l);
    hi[i] = h;
    lo[i] = l;
  }
}
__global__ void join_master_kernel(const __nv_bfloat16* __restrict__ hi, const short* __restrict__ lo,
                                   float* __restrict__ w, long long n) {
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n; i += (long long)gridDim.x * 256)
    w[i] = master_load(hi[i], lo[i]);
}

static int grid_for(long long n) {
  long long b = (n + 255) / 256;
  const long long cap = 148ll * 16;
  return (int)(b < cap ? (b < 1 ? 1 : b) : cap);
}

}  // namespace snu1

using namespace snu1;

// out[0] += sum g^2.  grad_dtype: 0 bf16, 1 fp32.
SNU1_API int snu1_sumsq(const void* g, long long n, int grad_dtype, float* out, void* stream) {
  if (n <= 0) return kHostOk;
  if (grad_dtype == 0)
    sumsq_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)g, n, out);
  else
    sumsq_kernel<float><<<grid_for(n), 256, 0, (cudaStream_t)stream>>>((const float*)g, n, out);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

// grad_dtype / state_dtype: 0 bf16, 1 fp32.
SNU1_API int snu1_adamw(void* p_hi, void* p_lo, const void* g, void* m, void* v, long long n,
                        int grad_dtype, int state_dtype, float lr, float beta1, float beta2,
                        float eps, float weight_decay, float bc1, float bc2, float grad_prescale,
                        const float* norm_sq, float max_norm, int* skipped, void* stream) {
  if (n <= 0) return kHostOk;
  if ((n & 7) != 0 || ((uintptr_t)p_hi & 15) || ((uintptr_t)p_lo & 15) || ((uintptr_t)g & 15) ||
      ((uintptr_t)m & 15) || ((uintptr_t)v & 15)) {
    set_last_error("adamw: ranges must be multiples of 8 elements and 16-byte aligned (n=%lld)", n);
    return kHostBadArg;
  }
  AdamArgs a;
  a.n = n;
  a.lr = lr;
  a.beta1 = beta1;
  a.beta2 = beta2;
  a.eps = eps;
  a.weight_decay = weight_decay;
  a.bc1 = bc1;
  a.bc2 = bc2;
  a.grad_prescale = grad_prescale;
  a.norm_sq = norm_sq;
  a.max_norm = max_norm;
  a.skipped = skipped;
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = grid_for(n >> 3);
  __nv_bfloat16* hi = (__nv_bfloat16*)p_hi;
  short* lo = (short*)p_lo;
  if (grad_dtype == 0 && state_dtype == 0)
    adamw_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, st>>>(hi, lo, (const __nv_bfloat16*)g,
                                                                     (__nv_bfloat16*)m, (__nv_bfloat16*)v, a);
  else if (grad_dtype == 0 && state_dtype == 1)
    adamw_kernel<__nv_bfloat16, float><<<grid, 256, 0, st>>>(hi, lo, (const __nv_bfloat16*)g, (float*)m,
                                                             (float*)v, a);
  else if (grad_dtype == 1 && state_dtype == 0)
    adamw_kernel<float, __nv_bfloat16><<<grid, 256, 0, st>>>(hi, lo, (const float*)g, (__nv_bfloat16*)m,
                                                             (__nv_bfloat16*)v, a);
  else
    adamw_kernel<float, float><<<grid, 256, 0, st>>>(hi, lo, (const float*)g, (float*)m, (float*)v, a);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_ema(float* ema, const void* p_hi, const void* p_lo, long long n, float decay,
                      void* stream) {
  if (n <= 0) return kHostOk;
  ema_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(ema, (const __nv_bfloat16*)p_hi,
                                                            (const short*)p_lo, n, decay);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_split_master(const float* w, void* hi, void* lo, long long n, void* stream) {
  if (n <= 0) return kHostOk;
  split_master_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>(w, (__nv_bfloat16*)hi, (short*)lo, n);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_join_master(const void* hi, const void* lo, float* w, long long n, void* stream) {
  if (n <= 0) return kHostOk;
  join_master_kernel<<<grid_for(n), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)hi,
                                                                    (const short*)lo, w, n);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

// ===========================================================================
// ZeRO-1 over NVLink peer memory: the collectives are done by the kernels.
//
// Gradient and parameter arenas live in symmetric memory (the same virtual layout
// on every GPU, every peer mapped).  Instead of NCCL reduce-scatter -> AdamW ->
// NCCL all-gather (reference: all-reduce + broadcast,
// training/sensenovalm/solver/optimizer/hybrid_zero_optim.py:626-690, 1033-1070):
//
//   zero_rs_sumsq    pulls this rank's piece of a bucket from every peer with plain
//                    peer loads, sums in fp32, leaves the reduced gradient in the local
//                    arena and adds its squared norm to the clip accumulator  (reduce-
//                    scatter + cast + norm in one pass);
//   zero_adamw_push  unscale + clip + AdamW on the fp32 master of the piece and stores
//                    the new bf16 weights straight into every peer's parameter arena
//                    (update + all-gather in one pass).
//
// Cross-GPU ordering uses flag words in symmetric memory: a producer stores a step
// counter with release semantics at system scope after its data, a consumer spins on
// it with acquire loads.  Every spin has a time limit and reports through the status
// word instead of hanging.  No multimem / multicast object is involved.
// ===========================================================================
namespace snu1 {

constexpr int kMaxPeers = 8;
struct PeerPtrs {
  void* p[kMaxPeers];
};

__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// flags layout on every rank: [slot][source rank]
__global__ void signal_peers_kernel(PeerPtrs flags, int world, int my_rank, int slot, int value) {
  __threadfence_system();
  const int r = threadIdx.x;
  if (r < world) st_release_sys(reinterpret_cast<int*>(flags.p[r]) + slot * world + my_rank, value);
}

// Waits (bounded) until every peer has published `value` in `slot`.  Returns false on timeout.
// `limit_ns` = 0 selects the built-in limit.
__device__ __forceinline__ bool wait_all_peers(const int* my_flags, int world, int slot, int value,
                                               int* status, int* s_fail, uint64_t limit_ns = 0) {
  const uint64_t limit = limit_ns ? limit_ns : kPeerWaitNs;
  if (threadIdx.x == 0) *s_fail = 0;
  __syncthreads();
  if (threadIdx.x < world) {
    const int* f = my_flags + slot * world + threadIdx.x;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (ld_acquire_sys(f) < value) {
      if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > limit) {
        *s_fail = 1;
        report_status(status, kPeerTimeout, 7);
        break;
      }
    }
  }
  __syncthreads();
  return *s_fail == 0;
}

__global__ void wait_flags_kernel(const int* my_flags, int world, int slot, int value, int* status,
                                  uint64_t limit_ns) {
  __shared__ int s_fail;
  wait_all_peers(my_flags, world, slot, value, status, &s_fail, limit_ns);
}

// Weight-parallel all-gather by peer loads: dst[r * per + i] = src_r[src_off + i] for every rank r (the local
// piece included), 16-byte vectors, eight independent loads in flight per thread so that a modest grid covers
// the NVLink latency-bandwidth product without taking the SMs from the GEMMs it runs beside.
__global__ void __launch_bounds__(256)
    wp_gather_kernel(PeerPtrs src, int world, long long src_off16, long long per16, uint4* __restrict__ dst) {
  constexpr int U = 8;
  const long long stride = (long long)gridDim.x * 256;
  for (int r = 0; r < world; ++r) {
    const uint4* s = reinterpret_cast<const uint4*>(src.p[r]) + src_off16;
    uint4* d = dst + (long long)r * per16;
    long long i = blockIdx.x * 256ll + threadIdx.x;
    for (; i + (U - 1) * stride < per16; i += U * stride) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) v[u] = s[i + u * stride];
#pragma unroll
      for (int u = 0; u < U; ++u) d[i + u * stride] = v[u];
    }
    for (; i < per16; i += stride) d[i] = s[i];
  }
}

// Reduce-scatter of one piece by peer loads from per-rank staging buffers: dst[i] (+)= sum_r src_r[src_off + i],
// fp32 sum, bf16 result, squared norm of what is stored added to norm_sq (when given).
__global__ void __launch_bounds__(256)
    rs_pull_kernel(PeerPtrs src, int world, long long src_off, long long n, __nv_bfloat16* __restrict__ dst,
                   int accumulate, float* norm_sq) {
  __shared__ float scratch[8];
  const long long nvec = n >> 3;
  float acc = 0.f;
  for (long long iv = blockIdx.x * 256ll + threadIdx.x; iv < nvec; iv += (long long)gridDim.x * 256) {
    float s[8];
    if (accumulate) {
      Vec8<__nv_bfloat16>::load(dst + (iv << 3), s);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) s[e] = 0.f;
    }
    for (int r = 0; r < world; ++r) {
      float f[8];
      Vec8<__nv_bfloat16>::load(reinterpret_cast<const __nv_bfloat16*>(src.p[r]) + src_off + (iv << 3), f);
#pragma unroll
      for (int e = 0; e < 8; ++e) s[e] += f[e];
    }
    Vec8<__nv_bfloat16>::store(dst + (iv << 3), s);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float rr = __bfloat162float(__float2bfloat16_rn(s[e]));
      acc += rr * rr;
    }
  }
  if (norm_sq == nullptr) return;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += scratch[i];
    atomicAdd(norm_sq, t);
  }
}

__global__ void __launch_bounds__(256)
    zero_rs_sumsq_kernel(PeerPtrs grads, int world, int my_rank, long long off, long long n,
                         const int* my_flags, int slot, int value, float* norm_sq, int* status) {
  __shared__ int s_fail;
  __shared__ float scratch[8];
  if (my_flags != nullptr && !wait_all_peers(my_flags, world, slot, value, status, &s_fail)) return;
  const long long nvec = n >> 3;
  float acc = 0.f;
  __nv_bfloat16* mine = reinterpret_cast<__nv_bfloat16*>(grads.p[my_rank]) + off;
  for (long long iv = blockIdx.x * 256ll + threadIdx.x; iv < nvec; iv += (long long)gridDim.x * 256) {
    float s[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) s[e] = 0.f;
    for (int r = 0; r < world; ++r) {
      float f[8];
      Vec8<__nv_bfloat16>::load(reinterpret_cast<const __nv_bfloat16*>(grads.p[r]) + off + (iv << 3), f);
#pragma unroll
      for (int e = 0; e < 8; ++e) s[e] += f[e];
    }
    Vec8<__nv_bfloat16>::store(mine + (iv << 3), s);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float rr = __bfloat162float(__float2bfloat16_rn(s[e]));  // norm of what is stored
      acc += rr * rr;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += scratch[i];
    atomicAdd(norm_sq, t);
  }
}

template <typename MT>
__global__ void __launch_bounds__(256)
    zero_adamw_push_kernel(PeerPtrs params, int world, int my_rank, long long off, short* __restrict__ p_lo,
                           const __nv_bfloat16* __restrict__ g, MT* __restrict__ m, MT* __restrict__ v,
                           const AdamArgs a) {
  float gscale = a.grad_prescale;
  bool skip = false;
  if (a.norm_sq != nullptr) {
    const float nsq = *a.norm_sq;
    if (!(nsq == nsq) || nsq > 3.0e38f) {
      if (blockIdx.x == 0 && threadIdx.x == 0 && a.skipped) *a.skipped = 1;
      skip = true;
    } else if (a.max_norm > 0.f) {
      const float coef = a.max_norm / (sqrtf(nsq) * a.grad_prescale + 1e-6f);
      if (coef < 1.f) gscale *= coef;
    }
  }
  if (skip) return;
  const float step = a.lr / a.bc1;
  const float inv_sqrt_bc2 = rsqrtf(a.bc2);
  const float decay = 1.f - a.lr * a.weight_decay;
  const long long nvec = a.n >> 3;
  __nv_bfloat16* p_hi = reinterpret_cast<__nv_bfloat16*>(params.p[my_rank]) + off;
  for (long long iv = blockIdx.x * 256ll + threadIdx.x; iv < nvec; iv += (long long)gridDim.x * 256) {
    const long long i = iv << 3;
    float gr[8], mi[8], vi[8];
    Vec8<__nv_bfloat16>::load(g + i, gr);
    Vec8<MT>::load(m + i, mi);
    Vec8<MT>::load(v + i, vi);
    const uint4 hu = *reinterpret_cast<const uint4*>(p_hi + i);
    const uint4 lu = *reinterpret_cast<const uint4*>(p_lo + i);
    const unsigned short* hs = reinterpret_cast<const unsigned short*>(&hu);
    const short* ls = reinterpret_cast<const short*>(&lu);
    uint4 ho, lo4;
    unsigned short* hos = reinterpret_cast<unsigned short*>(&ho);
    short* los = reinterpret_cast<short*>(&lo4);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float grad = gr[e] * gscale;
      float w = master_load(__ushort_as_bfloat16(hs[e]), ls[e]);
      mi[e] = a.beta1 * mi[e] + (1.f - a.beta1) * grad;
      vi[e] = a.beta2 * vi[e] + (1.f - a.beta2) * grad * grad;
      w = w * decay - step * (mi[e] / (sqrtf(vi[e]) * inv_sqrt_bc2 + a.eps));
      __nv_bfloat16 hi;
      short lo;
      master_store(w, hi, lo);
      hos[e] = __bfloat16_as_ushort(hi);
      los[e] = lo;
    }
    *reinterpret_cast<uint4*>(p_lo + i) = lo4;
    Vec8<MT>::store(m + i, mi);
    Vec8<MT>::store(v + i, vi);
    // all-gather by store: the new weights go to every rank's arena, this one included
    for (int r = 0; r < world; ++r)
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[r]) + off + i) = ho;
  }
}

// Stores `n16` 16-byte words from local `src` to byte offset `off` of the same buffer on every peer
// (the local copy included unless skip_self): the broadcast half of an all-gather, done with plain
// peer stores.
__global__ void __launch_bounds__(256)
    peer_put_kernel(const uint4* __restrict__ src, PeerPtrs dst, int world, int my_rank, long long off16,
                    long long n16, int skip_self) {
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n16; i += (long long)gridDim.x * 256) {
    const uint4 v = src[i];
    for (int r = 0; r < world; ++r) {
      if (skip_self && r == my_rank) continue;
      reinterpret_cast<uint4*>(dst.p[r])[off16 + i] = v;
    }
  }
}

// Plain 16-byte-vector copy; the source (or destination) may be a peer pointer.
__global__ void __launch_bounds__(256) copy16_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long n16) {
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n16; i += (long long)gridDim.x * 256) dst[i] = src[i];
}

static int fill_peers(PeerPtrs* out, const long long* ptrs, int world) {
  if (world < 1 || world > kMaxPeers) {
    set_last_error("peer kernels support 1..%d ranks (got %d)", kMaxPeers, world);
    return kHostBadArg;
  }
  for (int i = 0; i < kMaxPeers; ++i) out->p[i] = i < world ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return kHostOk;
}

}  // namespace snu1

SNU1_API int snu1_signal_peers(const long long* flag_ptrs, int world, int my_rank, int slot, int value,
                               void* stream) {
  PeerPtrs f;
  int rc = fill_peers(&f, flag_ptrs, world);
  if (rc != kHostOk) return rc;
  signal_peers_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(f, world, my_rank, slot, value);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

// Copies nbytes from src to dst with this package's own kernel (used to pull a peer's buffer into
// local memory: the source pointer may be a peer mapping).
SNU1_API int snu1_copy_bytes(const void* src, void* dst, long long nbytes, void* stream) {
  if (nbytes <= 0) return kHostOk;
  if ((nbytes & 15) || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) {
    set_last_error("copy_bytes: pointers and size must be multiples of 16 bytes");
    return kHostBadArg;
  }
  const long long n16 = nbytes >> 4;
  long long blocks = (n16 + 255) / 256;
  copy16_kernel<<<(int)(blocks < 1184 ? blocks : 1184), 256, 0, (cudaStream_t)stream>>>((const uint4*)src, (uint4*)dst, n16);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_peer_put(const void* src, const long long* dst_ptrs, int world, int my_rank, long long dst_off_bytes,
                           long long nbytes, int skip_self, void* stream) {
  if (nbytes <= 0) return kHostOk;
  if ((nbytes & 15) || (dst_off_bytes & 15) || (reinterpret_cast<uintptr_t>(src) & 15)) {
    set_last_error("peer_put: source, offset and size must be multiples of 16 bytes");
    return kHostBadArg;
  }
  PeerPtrs d;
  int rc = fill_peers(&d, dst_ptrs, world);
  if (rc != kHostOk) return rc;
  const long long n16 = nbytes >> 4;
  long long blocks = (n16 + 255) / 256;
  peer_put_kernel<<<(int)(blocks < 1184 ? blocks : 1184), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)src, d, world, my_rank, dst_off_bytes >> 4, n16, skip_self);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_wait_flags(const int* my_flags, int world, int slot, int value, void* stream) {
  wait_flags_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(my_flags, world, slot, value, device_status_word(), 0);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

// The same wait with the time limit as a launch argument (nanoseconds; 0 = the built-in limit).  When the limit runs
// out the kernel records kPeerTimeout in the status word and returns; the context stays usable.
SNU1_API int snu1_wait_flags_limit(const int* my_flags, int world, int slot, int value, long long limit_ns,
                                   void* stream) {
  if (limit_ns < 0) {
    set_last_error("wait_flags_limit: negative time limit");
    return kHostBadArg;
  }
  wait_flags_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(my_flags, world, slot, value, device_status_word(),
                                                        (uint64_t)limit_ns);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

// All-gather of one weight-parallel piece: every rank's `per` elements at element offset `src_off` of its shard
// buffer land at dst[r * per ...].  bf16 elements; offsets and sizes in multiples of 8 elements.
SNU1_API int snu1_wp_gather(const long long* src_ptrs, int world, long long src_off, long long per, void* dst,
                            int grid, void* stream) {
  if (per <= 0) return kHostOk;
  if ((per & 7) || (src_off & 7) || (reinterpret_cast<uintptr_t>(dst) & 15)) {
    set_last_error("wp_gather: offset, length (multiples of 8 elements) and destination (16 bytes) must be aligned");
    return kHostBadArg;
  }
  PeerPtrs p;
  int rc = fill_peers(&p, src_ptrs, world);
  if (rc != kHostOk) return rc;
  const long long per16 = per >> 3;
  long long blocks = (per16 + 255) / 256;
  if (grid <= 0) grid = 96;
  wp_gather_kernel<<<(int)(blocks < grid ? blocks : grid), 256, 0, (cudaStream_t)stream>>>(
      p, world, src_off >> 3, per16, reinterpret_cast<uint4*>(dst));
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

// Reduce-scatter pull of n bf16 elements from element offset src_off of every rank's staging buffer into dst
// (accumulate != 0: added to what dst holds).  norm_sq may be null.
SNU1_API int snu1_rs_pull(const long long* src_ptrs, int world, long long src_off, long long n, void* dst,
                          int accumulate, float* norm_sq, int grid, void* stream) {
  if (n <= 0) return kHostOk;
  if ((n & 7) || (src_off & 7) || (reinterpret_cast<uintptr_t>(dst) & 15)) {
    set_last_error("rs_pull: offset, length (multiples of 8 elements) and destination (16 bytes) must be aligned");
    return kHostBadArg;
  }
  PeerPtrs p;
  int rc = fill_peers(&p, src_ptrs, world);
  if (rc != kHostOk) return rc;
  long long blocks = ((n >> 3) + 255) / 256;
  if (grid <= 0) grid = 592;
  rs_pull_kernel<<<(int)(blocks < grid ? blocks : grid), 256, 0, (cudaStream_t)stream>>>(
      p, world, src_off, n, reinterpret_cast<__nv_bfloat16*>(dst), accumulate, norm_sq);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

// Reduce-scatter of one piece [off, off+n) by peer loads (+ squared norm).  my_flags may be
// null (no wait); otherwise the kernel first waits until every peer published `value` in `slot`.
SNU1_API int snu1_zero_rs_sumsq(const long long* grad_ptrs, int world, int my_rank, long long off,
                                long long n, const int* my_flags, int slot, int value, float* norm_sq,
                                void* stream) {
  if (n <= 0) return kHostOk;
  if ((n & 7) || (off & 7)) {
    set_last_error("zero_rs_sumsq: offset and length must be multiples of 8 elements");
    return kHostBadArg;
  }
  PeerPtrs g;
  int rc = fill_peers(&g, grad_ptrs, world);
  if (rc != kHostOk) return rc;
  long long blocks = ((n >> 3) + 255) / 256;
  const int grid = (int)(blocks < 592 ? blocks : 592);
  zero_rs_sumsq_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(g, world, my_rank, off, n, my_flags, slot,
                                                               value, norm_sq, device_status_word());
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_zero_adamw_push(const long long* param_ptrs, int world, int my_rank, long long off,
                                  void* p_lo, const void* g, void* m, void* v, long long n, int state_dtype,
                                  float lr, float beta1, float beta2, float eps, float weight_decay,
                                  float bc1, float bc2, float grad_prescale, const float* norm_sq,
                                  float max_norm, int* skipped, void* stream) {
  if (n <= 0) return kHostOk;
  if ((n & 7) || (off & 7)) {
    set_last_error("zero_adamw_push: offset and length must be multiples of 8 elements");
    return kHostBadArg;
  }
  PeerPtrs p;
  int rc = fill_peers(&p, param_ptrs, world);
  if (rc != kHostOk) return rc;
  AdamArgs a;
  a.n = n;
  a.lr = lr;
  a.beta1 = beta1;
  a.beta2 = beta2;
  a.eps = eps;
  a.weight_decay = weight_decay;
  a.bc1 = bc1;
  a.bc2 = bc2;
  a.grad_prescale = grad_prescale;
  a.norm_sq = norm_sq;
  a.max_norm = max_norm;
  a.skipped = skipped;
  const int grid = grid_for(n >> 3);
  cudaStream_t st = (cudaStream_t)stream;
  if (state_dtype == 0)
    zero_adamw_push_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p, world, my_rank, off, (short*)p_lo,
                                                                (const __nv_bfloat16*)g, (__nv_bfloat16*)m,
                                                                (__nv_bfloat16*)v, a);
  else
    zero_adamw_push_kernel<float><<<grid, 256, 0, st>>>(p, world, my_rank, off, (short*)p_lo,
                                                        (const __nv_bfloat16*)g, (float*)m, (float*)v, a);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}
