// packed_mixed_attention, backward, for sm_100a (tcgen05 / TMEM / TMA).
//
// Three kernels:
//   attn_delta   : delta[h][q] = sum_d dO * O  (one warp per row and head)
//   attn_bwd_dq  : a CTA owns 128 query rows of one head and walks its key tiles:
//                  S = Q K^T, dP = dO V^T (TMEM), dS = P * (dP - delta) * scale
//                  written as bf16 to shared memory, dQ += dS K (TMEM).
//   attn_bwd_dkv : a CTA owns 128 key rows of one KV head and walks (query tile,
//                  query head of the GQA group) pairs in 64-row sub-tiles:
//                  S^T = K Q^T, dP^T = V dO^T (double-buffered in TMEM),
//                  dV += P^T dO, dK += dS^T Q (TMEM).
// Recomputing S in both kernels costs two extra products per tile pair but needs
// no atomics, so gradients are deterministic.  The mask is evaluated only on
// tiles the classifier marked "partial".
//
// Reference: the backward of torch flex_attention used at
// training/sensenovalm/model/modules/mha.py:1548.
#include "attn_common.cuh"
#include "host_common.h"

namespace snu1 {
int encode_head_tmap(CUtensorMap* out, const void* base, long long rows, int heads, long long ld,
                     int box_rows);

namespace attn_bwd {

constexpr int HALF_BYTES = 128 * 64 * 2;    // 16 KB: 128 rows x 64 columns
constexpr int TILE_BYTES = 2 * HALF_BYTES;  // 32 KB
constexpr int SUB_HALF = 64 * 64 * 2;       // 8 KB: 64 rows x 64 columns
constexpr int SUB_TILE = 2 * SUB_HALF;      // 16 KB
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;

__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, long long ldo,
                                  const __nv_bfloat16* __restrict__ dout, long long lddo,
                                  float* __restrict__ delta, int Sq, int Hq) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= Sq * Hq) return;
  const int row = gw / Hq, h = gw - row * Hq;
  const uint2 a = *reinterpret_cast<const uint2*>(o + (long long)row * ldo + h * 128 + lane * 4);
  const uint2 b = *reinterpret_cast<const uint2*>(dout + (long long)row * lddo + h * 128 + lane * 4);
  float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
  float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
  float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.x));
  float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.y));
  float s = a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) delta[(long long)h * Sq + row] = s;
}

struct BwdArgs {
  const float* lse;    // [Hq][Sq] log2 domain
  const float* delta;  // [Hq][Sq]
  const TokMeta* meta_q;
  const TokMeta* meta_k;
  const int* list;   // dq: kv_list [nq][nk]; dkv: q_list [nk][nq]
  const int* count;  // dq: kv_count;        dkv: q_count
  const int* order;  // tile indices, longest list first (dq: query tiles; dkv: key tiles); may be null
  int list_stride;
  int Sq, Sk, Hq, Hkv;
  float scale, scale_log2;
  __nv_bfloat16* out0;  // dq   | dk
  long long ld0;
  __nv_bfloat16* out1;  //      | dv
  long long ld1;
  int* status;
  // mask bits of partial (query tile, key tile) pairs, written by the tile classifier; tile_slot may be null
  const int* tile_slot;   // [nq][nk_tiles] slot, -1 = none
  int nk_tiles;
  const uint32_t* bits_q;  // [slots][128 query rows][4 words]: dQ
  const uint32_t* bits_k;  // [slots][128 key rows][4 words]:   dK/dV
};

__device__ __forceinline__ void store_row_chunk(__nv_bfloat16* dst, const uint32_t (&r)[32]) {
  uint4* op = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 u;
    u.x = pack_bf16x2(__uint_as_float(r[i * 8 + 0]), __uint_as_float(r[i * 8 + 1]));
    u.y = pack_bf16x2(__uint_as_float(r[i * 8 + 2]), __uint_as_float(r[i * 8 + 3]));
    u.z = pack_bf16x2(__uint_as_float(r[i * 8 + 4]), __uint_as_float(r[i * 8 + 5]));
    u.w = pack_bf16x2(__uint_as_float(r[i * 8 + 6]), __uint_as_float(r[i * 8 + 7]));
    op[i] = u;
  }
}

// ------------------------------------ dQ ------------------------------------
// warp 0 TMA, warp 1 MMA, warps 2..9 element-wise: two warps per TMEM lane quarter, each
// owning 64 of the 128 key columns of a tile.
constexpr int DQ_THREADS = 320;

__global__ void __launch_bounds__(DQ_THREADS, 1)
    attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                       const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                       const BwdArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + TILE_BYTES;
  uint8_t* sK = sdO + TILE_BYTES;     // 2 stages
  uint8_t* sV = sK + 2 * TILE_BYTES;  // 2 stages
  uint8_t* sdS = sV + 2 * TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + TILE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;   // [2]
  uint64_t* kv_empty = bars + 3;  // [2]
  uint64_t* s_full = bars + 5;
  uint64_t* s_empty = bars + 6;
  uint64_t* dp_full = bars + 7;
  uint64_t* dp_empty = bars + 8;
  uint64_t* ds_full = bars + 9;
  uint64_t* ds_done = bars + 10;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x;   // heads fastest, tiles by ``order`` (longest list first)
  const int qt = args.order != nullptr ? args.order[blockIdx.y] : gridDim.y - 1 - blockIdx.y;
  const int kvh = head / (args.Hq / args.Hkv);
  const int q0 = qt * 128;
  const int n = args.count[qt];
  const int* list = args.list + (long long)qt * args.list_stride;

  if (n == 0) {
    if (warp >= 2 && warp < 6) {
      const int row = q0 + (warp - 2) * 32 + lane;
      if (row < args.Sq) {
        uint4 z = make_uint4(0, 0, 0, 0);
        uint4* op = reinterpret_cast<uint4*>(args.out0 + (long long)row * args.ld0 + head * 128);
#pragma unroll
        for (int i = 0; i < 16; ++i) op[i] = z;
      }
    }
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_empty, 8);
    mbar_init(dp_full, 1);
    mbar_init(dp_empty, 8);
    mbar_init(ds_full, 8);
    mbar_init(ds_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base, tmem_dP = tmem_base + 128, tmem_dQ = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, 2 * TILE_BYTES);
      tma_load_3d(sQ, &tmQ, q_full, 0, head, q0);
      tma_load_3d(sQ + HALF_BYTES, &tmQ, q_full, 64, head, q0);
      tma_load_3d(sdO, &tmdO, q_full, 0, head, q0);
      tma_load_3d(sdO + HALF_BYTES, &tmdO, q_full, 64, head, q0);
      int next_entry = list[0];   // fetched one iteration ahead: no global load between a free slot and its TMA
      for (int j = 0; j < n; ++j) {
        const int s = j & 1;
        const int k0 = list_tile(next_entry) * 128;
        if (j + 1 < n) next_entry = list[j + 1];
        if (!mbar_wait(&kv_empty[s], ((j >> 1) & 1) ^ 1, abort_flag, args.status, 1)) break;
        mbar_expect_tx(&kv_full[s], 2 * TILE_BYTES);
        tma_load_3d(sK + s * TILE_BYTES, &tmK, &kv_full[s], 0, kvh, k0);
        tma_load_3d(sK + s * TILE_BYTES + HALF_BYTES, &tmK, &kv_full[s], 64, kvh, k0);
        tma_load_3d(sV + s * TILE_BYTES, &tmV, &kv_full[s], 0, kvh, k0);
        tma_load_3d(sV + s * TILE_BYTES + HALF_BYTES, &tmV, &kv_full[s], 64, kvh, k0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_kk = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_kmn = make_idesc_bf16(128, 128, false, true);
      const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sdO), ds_addr = smem_u32(sdS);
      bool ok = mbar_wait(q_full, 0, abort_flag, args.status, 3);
      auto issue_s = [&](int j) {
        const uint32_t k_addr = smem_u32(sK + (j & 1) * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
          umma_bf16_ss(tmem_S, make_smem_desc(q_addr + off, 0, 1024),
                       make_smem_desc(k_addr + off, 0, 1024), idesc_kk, k > 0 ? 1u : 0u);
        }
        umma_commit(s_full);
      };
      auto issue_dp = [&](int j) {
        const uint32_t v_addr = smem_u32(sV + (j & 1) * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
          umma_bf16_ss(tmem_dP, make_smem_desc(do_addr + off, 0, 1024),
                       make_smem_desc(v_addr + off, 0, 1024), idesc_kk, k > 0 ? 1u : 0u);
        }
        umma_commit(dp_full);
      };
      // Two independent queues: S / dP of key tile `next_s` (needs the tile loaded and the S / dP TMEM
      // buffers drained) and dQ of key tile `next_dq` (needs dS written).  They are issued in whichever
      // order their inputs become ready: a K / V slot is only released by the dQ product that reads it, so
      // waiting for the next tile's load before issuing the dQ product that is already possible (the
      // former fixed order) left the load latency exposed in every iteration.
      int next_s = 0, next_dq = 0;
      uint64_t t_idle = 0;
      uint32_t spins = 0;
      while (ok && next_dq < n) {
        bool progressed = false;
        if (next_s < n && next_s <= next_dq + 1) {
          const int j = next_s;
          const bool s_free = j == 0 || mbar_try_wait(s_empty, (j - 1) & 1);
          const bool dp_free = j == 0 || mbar_try_wait(dp_empty, (j - 1) & 1);
          if (s_free && dp_free && mbar_try_wait(&kv_full[j & 1], (j >> 1) & 1)) {
            tc_fence_after();
            issue_s(j);
            issue_dp(j);
            ++next_s;
            progressed = true;
          }
        }
        if (next_dq < next_s && mbar_try_wait(ds_full, next_dq & 1)) {
          const int j = next_dq;
          tc_fence_after();
          const uint32_t k_addr = smem_u32(sK + (j & 1) * TILE_BYTES);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t a_off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
            umma_bf16_ss(tmem_dQ, make_smem_desc(ds_addr + a_off, 0, 1024),
                         make_smem_desc(k_addr + k * 2048, HALF_BYTES, 1024), idesc_kmn,
                         (j > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&kv_empty[j & 1]);
          umma_commit(ds_done);
          ++next_dq;
          progressed = true;
        }
        if (progressed) {
          t_idle = 0;
          spins = 0;
        } else if ((++spins & 0x3ff) == 0) {
          // bounded: nothing became ready for kLocalWaitNs -> report and let every role drain
          if (*abort_flag) {
            ok = false;
          } else if (t_idle == 0) {
            t_idle = globaltimer_ns();
          } else if (globaltimer_ns() - t_idle > kLocalWaitNs) {
            *abort_flag = 1;
            report_status(args.status, kWaitTimeout, 2);
            ok = false;
          }
        }
      }
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;  // which 64 key columns
    const int rloc = quarter * 32 + lane;
    const int row = q0 + rloc;
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    const bool row_ok = row < args.Sq;
    TokMeta mq = row_ok ? args.meta_q[row] : TokMeta{-1, 0, 0, 0};
    const float lse = row_ok ? args.lse[(long long)head * args.Sq + row] : __int_as_float(0x7f800000);
    const float dl = row_ok ? args.delta[(long long)head * args.Sq + row] : 0.f;
    const float sc2 = args.scale_log2, sc = args.scale;
    bool ok = true;
    for (int j = 0; j < n && ok; ++j) {
      const int entry = list[j];
      const bool partial = list_class(entry) != kTileFull;
      const int k0 = list_tile(entry) * 128 + half * 64;
      if (!mbar_wait(s_full, j & 1, abort_flag, args.status, 5)) {
        ok = false;
        break;
      }
      tc_fence_after();
      float p[64];
      {
        uint32_t r0[32], r1[32];
        const uint32_t ta = tmem_S + half * 64 + lane_sel;
        tmem_ld_32x32b_x32(ta, r0);
        tmem_ld_32x32b_x32(ta + 32, r1);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          p[c] = __uint_as_float(r0[c]);
          p[32 + c] = __uint_as_float(r1[c]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty);
      if (partial) {
        uint32_t w[2];
        const int slot =
            args.tile_slot != nullptr ? __ldg(args.tile_slot + (long long)qt * args.nk_tiles + list_tile(entry)) : -1;
        if (slot >= 0) {
          const uint2 u = __ldg(reinterpret_cast<const uint2*>(args.bits_q) + ((long long)slot * 128 + rloc) * 2 + half);
          w[0] = u.x;
          w[1] = u.y;
        } else {
          mask_words_by_rule<2>(mq, args.meta_k + k0, args.Sk - k0, true, w);
        }
#pragma unroll
        for (int g = 0; g < 2; ++g) {   // words that are uniform over the warp's rows need no per-element test
          if (__all_sync(0xffffffffu, w[g] == 0xffffffffu)) continue;
          if (__all_sync(0xffffffffu, w[g] == 0u)) {
#pragma unroll
            for (int c = 0; c < 32; ++c) p[g * 32 + c] = -INFINITY;
          } else {
#pragma unroll
            for (int c = 0; c < 32; ++c)
              if (!((w[g] >> c) & 1u)) p[g * 32 + c] = -INFINITY;
          }
        }
      }
      {
        const uint64_t sc2p = pack_f32x2(sc2, sc2), nl = pack_f32x2(-lse, -lse);
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(p[c], p[c + 1]), sc2p, nl), x0, x1);
          p[c] = fast_exp2(x0);
          p[c + 1] = fast_exp2(x1);
        }
      }
      if (!mbar_wait(dp_full, j & 1, abort_flag, args.status, 5)) {
        ok = false;
        break;
      }
      if (j > 0 && !mbar_wait(ds_done, (j - 1) & 1, abort_flag, args.status, 5)) {
        ok = false;
        break;
      }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_dP + half * 64 + c * 32 + lane_sel, r);
        tmem_ld_wait();
        if (c == 1) {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(dp_empty);
        }
        const uint64_t scp = pack_f32x2(sc, sc), ndl = pack_f32x2(-dl * sc, -dl * sc);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float d[8];
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            // dS = p * (dP * scale - delta * scale)
            const uint64_t u2 = fma_f32x2(pack_f32x2(__uint_as_float(r[i * 8 + e]), __uint_as_float(r[i * 8 + e + 1])), scp, ndl);
            unpack_f32x2(mul_f32x2(pack_f32x2(p[c * 32 + i * 8 + e], p[c * 32 + i * 8 + e + 1]), u2), d[e], d[e + 1]);
          }
          uint4 u;
          u.x = pack_bf16x2(d[0], d[1]);
          u.y = pack_bf16x2(d[2], d[3]);
          u.z = pack_bf16x2(d[4], d[5]);
          u.w = pack_bf16x2(d[6], d[7]);
          // this thread's 64 columns are exactly one 64-column box (index `half`)
          *reinterpret_cast<uint4*>(sdS + half * HALF_BYTES + swz128_offset(rloc, c * 4 + i)) = u;
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    if (ok && mbar_wait(ds_done, (n - 1) & 1, abort_flag, args.status, 5)) {
      tc_fence_after();
#pragma unroll 1
      for (int c = half * 2; c < half * 2 + 2; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_dQ + c * 32 + lane_sel, r);
        tmem_ld_wait();
        if (row_ok) store_row_chunk(args.out0 + (long long)row * args.ld0 + head * 128 + c * 32, r);
        __syncwarp();
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 2000000ull) {
      }
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}
constexpr int DQ_SMEM = 7 * TILE_BYTES + 256 + 1024;

// ---------------------------------- dK, dV ----------------------------------
// warp 0: TMA producer (also stages lse / delta of the query sub-tile in shared memory)
// warp 1: MMA issuer; warps 2..9: element-wise.  Two element-wise warps share each TMEM
// lane quarter and split the 64 query columns of a sub-tile between them.
constexpr int DKV_THREADS = 320;
constexpr int DKV_STAGES = 3;  // Q / dO sub-tile ring depth (4 would exceed 227 KB by a few hundred bytes)

__global__ void __launch_bounds__(DKV_THREADS, 1)
    attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                        const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                        const BwdArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE_BYTES;
  // Q / dO sub-tiles ride a DKV_STAGES-deep ring: a slot is only released when the dV / dK MMAs that
  // read it have completed, so with two slots the global-load latency of the next sub-tile (lse / delta
  // loads + TMA) sat exposed in every iteration; a deeper ring keeps loads in flight behind the MMAs.
  uint8_t* sQ = sV + TILE_BYTES;                // DKV_STAGES x 16 KB
  uint8_t* sdO = sQ + DKV_STAGES * SUB_TILE;    // DKV_STAGES x 16 KB
  uint8_t* sPT = sdO + DKV_STAGES * SUB_TILE;   // 16 KB: [128 key rows][64 queries]
  uint8_t* sdST = sPT + HALF_BYTES;             // 16 KB
  float* sLse = reinterpret_cast<float*>(sdST + HALF_BYTES);  // [DKV_STAGES][64]
  float* sDl = sLse + DKV_STAGES * 64;                         // [DKV_STAGES][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDl + DKV_STAGES * 64);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;                    // [DKV_STAGES]
  uint64_t* qdo_empty = qdo_full + DKV_STAGES;      // [DKV_STAGES]
  uint64_t* sdp_full = qdo_empty + DKV_STAGES;      // [2]
  uint64_t* sdp_empty = sdp_full + 2;               // [2]
  uint64_t* pds_full = sdp_empty + 2;
  uint64_t* pds_done = pds_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pds_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.x;
  const int kt = args.order != nullptr ? args.order[blockIdx.y] : blockIdx.y;
  const int rep = args.Hq / args.Hkv;
  const int k0 = kt * 128;
  const int nq_tiles = args.count[kt];
  const int n = nq_tiles * rep * 2;  // iterations: (query tile, head in group, 64-row half)
  const int* list = args.list + (long long)kt * args.list_stride;

  if (n == 0) {
    if (warp >= 2 && warp < 6) {
      const int row = k0 + (warp - 2) * 32 + lane;
      if (row < args.Sk) {
        uint4 z = make_uint4(0, 0, 0, 0);
        uint4* o0 = reinterpret_cast<uint4*>(args.out0 + (long long)row * args.ld0 + kvh * 128);
        uint4* o1 = reinterpret_cast<uint4*>(args.out1 + (long long)row * args.ld1 + kvh * 128);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          o0[i] = z;
          o1[i] = z;
        }
      }
    }
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < DKV_STAGES; ++i) {
      mbar_init(&qdo_full[i], 2);
      mbar_init(&qdo_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sdp_full[i], 1);
      mbar_init(&sdp_empty[i], 8);
    }
    mbar_init(pds_full, 8);
    mbar_init(pds_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // columns: S^T buffers [0,64) [64,128); dP^T buffers [128,192) [192,256); dV [256,384); dK [384,512)
  const uint32_t tmem_ST = tmem_base, tmem_dPT = tmem_base + 128;
  const uint32_t tmem_dV = tmem_base + 256, tmem_dK = tmem_base + 384;

  // iteration -> (query row start, query head, list entry)
  auto decode = [&](int i, int& qrow0, int& qh, int& entry) {
    const int e = i / (2 * rep);
    const int rem = i - e * 2 * rep;
    entry = list[e];
    qh = kvh * rep + (rem >> 1);
    qrow0 = list_tile(entry) * 128 + (rem & 1) * 64;
  };

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * TILE_BYTES);
      tma_load_3d(sK, &tmK, kv_full, 0, kvh, k0);
      tma_load_3d(sK + HALF_BYTES, &tmK, kv_full, 64, kvh, k0);
      tma_load_3d(sV, &tmV, kv_full, 0, kvh, k0);
      tma_load_3d(sV + HALF_BYTES, &tmV, kv_full, 64, kvh, k0);
    }
    // The loads of sub-tile i + 1 that do not need a free ring slot (its list entry, then its log-sum-exp and
    // delta values) are issued one iteration ahead into registers, and the TMA copies of a sub-tile start
    // before those values are stored: a slot's reload costs one TMA latency instead of two dependent global
    // loads plus the TMA latency.  qdo_full counts two arrivals: the expect-tx one and the one after the stores.
    bool ok = true;
    float pl[2], pd[2];
    int qrow0, qh, entry;
    auto fetch = [&](int i) {
      decode(i, qrow0, qh, entry);
      const float* lse_p = args.lse + (long long)qh * args.Sq;
      const float* dl_p = args.delta + (long long)qh * args.Sq;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int c = lane + 32 * h;
        const bool in = qrow0 + c < args.Sq;
        // kept negated (and delta pre-multiplied by the softmax scale): they are the addends of the packed
        // FMAs in the element-wise warps; -inf past the end makes p = 0 there
        pl[h] = in ? -__ldg(lse_p + qrow0 + c) : __int_as_float(0xff800000);
        pd[h] = in ? -__ldg(dl_p + qrow0 + c) * args.scale : 0.f;
      }
    };
    fetch(0);
    for (int i = 0; i < n; ++i) {
      const int s = i % DKV_STAGES;
      if (lane == 0) ok = mbar_wait(&qdo_empty[s], ((i / DKV_STAGES) & 1) ^ 1, abort_flag, args.status, 1);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(&qdo_full[s], 2 * SUB_TILE);
        tma_load_3d(sQ + s * SUB_TILE, &tmQ, &qdo_full[s], 0, qh, qrow0);
        tma_load_3d(sQ + s * SUB_TILE + SUB_HALF, &tmQ, &qdo_full[s], 64, qh, qrow0);
        tma_load_3d(sdO + s * SUB_TILE, &tmdO, &qdo_full[s], 0, qh, qrow0);
        tma_load_3d(sdO + s * SUB_TILE + SUB_HALF, &tmdO, &qdo_full[s], 64, qh, qrow0);
      }
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        sLse[s * 64 + lane + 32 * h] = pl[h];
        sDl[s * 64 + lane + 32 * h] = pd[h];
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&qdo_full[s]);
      if (i + 1 < n) fetch(i + 1);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_st = make_idesc_bf16(128, 64, false, false);
      constexpr uint32_t idesc_acc = make_idesc_bf16(128, 128, false, true);
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      const uint32_t pt_addr = smem_u32(sPT), dst_addr = smem_u32(sdST);
      bool ok = mbar_wait(kv_full, 0, abort_flag, args.status, 3);
      auto issue_sdp = [&](int i) {
        const int s = i & 1, qs = i % DKV_STAGES;
        const uint32_t q_addr = smem_u32(sQ + qs * SUB_TILE), do_addr = smem_u32(sdO + qs * SUB_TILE);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t a_off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
          const uint32_t b_off = (k >> 2) * SUB_HALF + (k & 3) * 32;
          umma_bf16_ss(tmem_ST + s * 64, make_smem_desc(k_addr + a_off, 0, 1024),
                       make_smem_desc(q_addr + b_off, 0, 1024), idesc_st, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t a_off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
          const uint32_t b_off = (k >> 2) * SUB_HALF + (k & 3) * 32;
          umma_bf16_ss(tmem_dPT + s * 64, make_smem_desc(v_addr + a_off, 0, 1024),
                       make_smem_desc(do_addr + b_off, 0, 1024), idesc_st, k > 0 ? 1u : 0u);
        }
        umma_commit(&sdp_full[s]);
      };
      // Two queues, issued in whichever order their inputs become ready: S^T / dP^T of sub-tile `next_s`
      // (needs its Q / dO slot loaded and its TMEM buffers drained; at most two ahead of the dV / dK queue,
      // one per TMEM buffer) and dV / dK of sub-tile `next_acc` (needs P^T / dS^T written).  A Q / dO slot is
      // only released by the dV / dK products that read it, so waiting for the next sub-tile's load before
      // issuing products that are already possible would delay that very release.
      int next_s = 0, next_acc = 0;
      uint64_t t_idle = 0;
      uint32_t spins = 0;
      while (ok && next_acc < n) {
        bool progressed = false;
        if (next_s < n && next_s <= next_acc + 1) {
          const int i = next_s;
          if (mbar_try_wait(&sdp_empty[i & 1], ((i >> 1) & 1) ^ 1) &&
              mbar_try_wait(&qdo_full[i % DKV_STAGES], (i / DKV_STAGES) & 1)) {
            tc_fence_after();
            issue_sdp(i);
            ++next_s;
            progressed = true;
          }
        }
        if (next_acc < next_s && mbar_try_wait(pds_full, next_acc & 1)) {
          const int i = next_acc;
          tc_fence_after();
          const int qs = i % DKV_STAGES;
          const uint32_t q_addr = smem_u32(sQ + qs * SUB_TILE), do_addr = smem_u32(sdO + qs * SUB_TILE);
#pragma unroll
          for (int k = 0; k < 4; ++k) {  // reduction over the 64 query rows
            umma_bf16_ss(tmem_dV, make_smem_desc(pt_addr + k * 32, 0, 1024),
                         make_smem_desc(do_addr + k * 2048, SUB_HALF, 1024), idesc_acc,
                         (i > 0 || k > 0) ? 1u : 0u);
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            umma_bf16_ss(tmem_dK, make_smem_desc(dst_addr + k * 32, 0, 1024),
                         make_smem_desc(q_addr + k * 2048, SUB_HALF, 1024), idesc_acc,
                         (i > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&qdo_empty[qs]);
          umma_commit(pds_done);
          ++next_acc;
          progressed = true;
        }
        if (progressed) {
          t_idle = 0;
          spins = 0;
        } else if ((++spins & 0x3ff) == 0) {
          // bounded: nothing became ready for kLocalWaitNs -> report and let every role drain
          if (*abort_flag) {
            ok = false;
          } else if (t_idle == 0) {
            t_idle = globaltimer_ns();
          } else if (globaltimer_ns() - t_idle > kLocalWaitNs) {
            *abort_flag = 1;
            report_status(args.status, kWaitTimeout, 2);
            ok = false;
          }
        }
      }
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;      // which 32 query columns of the sub-tile
    const int rloc = quarter * 32 + lane;  // key row inside the tile
    const int krow = k0 + rloc;
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    const bool krow_ok = krow < args.Sk;
    const bool tile_rows_ok = k0 + 128 <= args.Sk;
    TokMeta mk = krow_ok ? args.meta_k[krow] : TokMeta{-2, 0, 0, kFlagBlocked};
    const float sc2 = args.scale_log2, sc = args.scale;
    bool ok = true;
    for (int i = 0; i < n && ok; ++i) {
      const int s = i & 1;
      int qrow0, qh, entry;
      decode(i, qrow0, qh, entry);
      const bool fast = list_class(entry) == kTileFull && tile_rows_ok;
      if (!mbar_wait(&sdp_full[s], (i >> 1) & 1, abort_flag, args.status, 5)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t st[32], dp[32];
      tmem_ld_32x32b_x32(tmem_ST + s * 64 + half * 32 + lane_sel, st);
      tmem_ld_32x32b_x32(tmem_dPT + s * 64 + half * 32 + lane_sel, dp);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sdp_empty[s]);
      const int qs = i % DKV_STAGES;
      const float* lse_s = sLse + qs * 64 + half * 32;
      const float* dl_s = sDl + qs * 64 + half * 32;
      uint32_t pk[16], dk[16];
      const uint64_t sc2p = pack_f32x2(sc2, sc2), scp = pack_f32x2(sc, sc);
      uint32_t allow_w[1] = {0xffffffffu};
      if (!fast) {
        const int slot = args.tile_slot != nullptr
                             ? __ldg(args.tile_slot + (long long)(qrow0 >> 7) * args.nk_tiles + kt)
                             : -1;
        if (slot >= 0)
          allow_w[0] = __ldg(args.bits_k + ((long long)slot * 128 + rloc) * 4 + ((qrow0 & 127) >> 5) + half);
        else if (krow_ok)
          mask_words_by_rule<1>(mk, args.meta_q + qrow0 + half * 32, args.Sq - qrow0 - half * 32, false, allow_w);
        else
          allow_w[0] = 0u;
      }
      {
        const uint32_t aw = allow_w[0];
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          // p = 2^(s * scale_log2 - lse), dS = p * (dP * scale - delta * scale): three packed fp32 ops,
          // two exponentials and two conversions per pair of elements
          const uint64_t nl = *reinterpret_cast<const uint64_t*>(lse_s + c);
          const uint64_t nd = *reinterpret_cast<const uint64_t*>(dl_s + c);
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(st[c]), __uint_as_float(st[c + 1])), sc2p, nl), x0, x1);
          const float p0 = ((aw >> c) & 1u) ? fast_exp2(x0) : 0.f;
          const float p1 = ((aw >> (c + 1)) & 1u) ? fast_exp2(x1) : 0.f;
          const uint64_t u = fma_f32x2(pack_f32x2(__uint_as_float(dp[c]), __uint_as_float(dp[c + 1])), scp, nd);
          float d0, d1;
          unpack_f32x2(mul_f32x2(pack_f32x2(p0, p1), u), d0, d1);
          pk[c >> 1] = pack_bf16x2(p0, p1);
          dk[c >> 1] = pack_bf16x2(d0, d1);
        }
      }
      if (i > 0 && !mbar_wait(pds_done, (i - 1) & 1, abort_flag, args.status, 5)) {
        ok = false;
        break;
      }
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        const uint32_t off = swz128_offset(rloc, half * 4 + ch);
        *reinterpret_cast<uint4*>(sPT + off) = make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
        *reinterpret_cast<uint4*>(sdST + off) = make_uint4(dk[ch * 4], dk[ch * 4 + 1], dk[ch * 4 + 2], dk[ch * 4 + 3]);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
    }
    if (ok && mbar_wait(pds_done, (n - 1) & 1, abort_flag, args.status, 5)) {
      tc_fence_after();
      // each of the two warps of a lane quarter writes half of the 128 output columns
#pragma unroll 1
      for (int c = half * 2; c < half * 2 + 2; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_dV + c * 32 + lane_sel, r);
        tmem_ld_wait();
        if (krow_ok) store_row_chunk(args.out1 + (long long)krow * args.ld1 + kvh * 128 + c * 32, r);
        __syncwarp();
        tmem_ld_32x32b_x32(tmem_dK + c * 32 + lane_sel, r);
        tmem_ld_wait();
        if (krow_ok) store_row_chunk(args.out0 + (long long)krow * args.ld0 + kvh * 128 + c * 32, r);
        __syncwarp();
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 2000000ull) {
      }
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}
constexpr int DKV_SMEM = 2 * TILE_BYTES + 2 * DKV_STAGES * SUB_TILE + 2 * HALF_BYTES + DKV_STAGES * 512 + 256 + 1024;
static_assert(DKV_SMEM <= 227 * 1024, "dK/dV kernel exceeds the shared memory of one CTA");

}  // namespace attn_bwd
}  // namespace snu1

using namespace snu1;

// dq [Sq,Hq,128], dk/dv [Sk,Hkv,128] (row strides ld*), all bf16.  delta is scratch [Hq][Sq] fp32.
SNU1_API int snu1_attn_bwd(const void* q, long long ldq, const void* k, long long ldk, const void* v,
                           long long ldv, const void* o, long long ldo, const void* dout,
                           long long lddo, const float* lse, float* delta, void* dq, long long lddq,
                           void* dk, long long lddk, void* dv, long long lddv, const void* meta_q,
                           const void* meta_k, const int* kv_list, const int* kv_count,
                           const int* q_list, const int* q_count, int Sq, int Sk, int Hq, int Hkv,
                           float scale, const int* tile_slot, const void* bits_q, const void* bits_k,
                           const int* q_order, const int* kv_order, void* stream) {
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || Sq <= 0 || Sk <= 0) {
    set_last_error("attn_bwd: bad head counts / lengths");
    return kHostBadArg;
  }
  if (ldq % 8 || ldk % 8 || ldv % 8 || ldo % 8 || lddo % 8 || lddq % 8 || lddk % 8 || lddv % 8) {
    set_last_error("attn_bwd: row strides must be multiples of 8 elements");
    return kHostBadArg;
  }
  cudaStream_t st = (cudaStream_t)stream;
  const int nq = (Sq + 127) / 128, nk = (Sk + 127) / 128;
  {
    const long long warps = (long long)Sq * Hq;
    const int blocks = (int)((warps * 32 + 255) / 256);
    attn_bwd::attn_delta_kernel<<<blocks, 256, 0, st>>>((const __nv_bfloat16*)o, ldo,
                                                        (const __nv_bfloat16*)dout, lddo, delta, Sq, Hq);
  }
  CUtensorMap tmQ, tmdO, tmK, tmV, tmQ64, tmdO64;
  int rc;
  if ((rc = encode_head_tmap(&tmQ, q, Sq, Hq, ldq, 128)) != kHostOk) return rc;
  if ((rc = encode_head_tmap(&tmdO, dout, Sq, Hq, lddo, 128)) != kHostOk) return rc;
  if ((rc = encode_head_tmap(&tmQ64, q, Sq, Hq, ldq, 64)) != kHostOk) return rc;
  if ((rc = encode_head_tmap(&tmdO64, dout, Sq, Hq, lddo, 64)) != kHostOk) return rc;
  if ((rc = encode_head_tmap(&tmK, k, Sk, Hkv, ldk, 128)) != kHostOk) return rc;
  if ((rc = encode_head_tmap(&tmV, v, Sk, Hkv, ldv, 128)) != kHostOk) return rc;
  attn_bwd::BwdArgs a;
  a.lse = lse;
  a.delta = delta;
  a.meta_q = (const TokMeta*)meta_q;
  a.meta_k = (const TokMeta*)meta_k;
  a.Sq = Sq;
  a.Sk = Sk;
  a.Hq = Hq;
  a.Hkv = Hkv;
  a.scale = scale;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = device_status_word();
  a.tile_slot = (bits_q != nullptr && bits_k != nullptr) ? tile_slot : nullptr;
  a.nk_tiles = nk;
  a.bits_q = (const uint32_t*)bits_q;
  a.bits_k = (const uint32_t*)bits_k;
  // dQ
  a.list = kv_list;
  a.count = kv_count;
  a.list_stride = nk;
  a.order = q_order;
  a.out0 = (__nv_bfloat16*)dq;
  a.ld0 = lddq;
  a.out1 = nullptr;
  a.ld1 = 0;
  SNU1_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd::attn_bwd_dq_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       attn_bwd::DQ_SMEM));
  attn_bwd::attn_bwd_dq_kernel<<<dim3(Hq, nq), attn_bwd::DQ_THREADS, attn_bwd::DQ_SMEM, st>>>(
      tmQ, tmdO, tmK, tmV, a);
  // dK, dV
  a.list = q_list;
  a.count = q_count;
  a.list_stride = nq;
  a.order = kv_order;
  a.out0 = (__nv_bfloat16*)dk;
  a.ld0 = lddk;
  a.out1 = (__nv_bfloat16*)dv;
  a.ld1 = lddv;
  SNU1_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd::attn_bwd_dkv_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       attn_bwd::DKV_SMEM));
  attn_bwd::attn_bwd_dkv_kernel<<<dim3(Hkv, nk), attn_bwd::DKV_THREADS, attn_bwd::DKV_SMEM, st>>>(
      tmQ64, tmdO64, tmK, tmV, a);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

// ---------------------------------------------------------------------------
// Allocation-free variant (declared and documented in snu1_noalloc.h).
// The scratch lives in the library image; host code only ever uses the device
// address obtained from cudaGetSymbolAddress, never the symbol itself.
// ---------------------------------------------------------------------------
#include "snu1_noalloc.h"

namespace snu1 {
namespace {
constexpr size_t kNoAllocStatusBytes = 256;  // status word, padded to keep delta 256-byte aligned
static __device__ __align__(256) unsigned char
    g_noalloc_scratch[kNoAllocStatusBytes + sizeof(float) * SNU1_NOALLOC_MAX_DELTA];

constexpr int kNoAllocMaxDevices = 64;
void* g_noalloc_addr[kNoAllocMaxDevices] = {nullptr};

// Device address of the scratch on the current device; looked up once per device.
int noalloc_scratch(unsigned char** out) {
  int dev = 0;
  SNU1_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kNoAllocMaxDevices) {
    set_last_error("attn_bwd_noalloc: device index %d out of range", dev);
    return kHostBadArg;
  }
  if (g_noalloc_addr[dev] == nullptr) {
    void* p = nullptr;
    SNU1_CUDA_CHECK(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    g_noalloc_addr[dev] = p;
  }
  *out = static_cast<unsigned char*>(g_noalloc_addr[dev]);
  return kHostOk;
}
}  // namespace
}  // namespace snu1

SNU1_API int snu1_attn_bwd_noalloc(const void* q, long long ldq, const void* k, long long ldk,
                                   const void* v, long long ldv, const void* o, long long ldo,
                                   const void* dout, long long lddo, const float* lse, void* dq,
                                   long long lddq, void* dk, long long lddk, void* dv, long long lddv,
                                   const void* meta_q, const void* meta_k, const int* kv_list,
                                   const int* kv_count, const int* q_list, const int* q_count, int Sq,
                                   int Sk, int Hq, int Hkv, float scale, int* status_out, void* stream) {
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || Sq <= 0 || Sk <= 0) {
    set_last_error("attn_bwd_noalloc: bad head counts / lengths");
    return kHostBadArg;
  }
  if ((long long)Hq * Sq > (long long)SNU1_NOALLOC_MAX_DELTA) {
    set_last_error("attn_bwd_noalloc: Hq * Sq = %lld exceeds the built-in scratch of %d floats; "
                   "use snu1_attn_bwd with caller-provided scratch for this size",
                   (long long)Hq * Sq, SNU1_NOALLOC_MAX_DELTA);
    return SNU1_NOALLOC_TOO_LARGE;
  }
  if (ldq % 8 || ldk % 8 || ldv % 8 || ldo % 8 || lddo % 8 || lddq % 8 || lddk % 8 || lddv % 8) {
    set_last_error("attn_bwd_noalloc: row strides must be multiples of 8 elements");
    return kHostBadArg;
  }
  unsigned char* scratch = nullptr;
  int rc = noalloc_scratch(&scratch);
  if (rc != kHostOk) return rc;
  int* status = reinterpret_cast<int*>(scratch);
  float* delta = reinterpret_cast<float*>(scratch + kNoAllocStatusBytes);
  cudaStream_t st = (cudaStream_t)stream;
  const int nq = (Sq + 127) / 128, nk = (Sk + 127) / 128;
  // the status word is the only part that has to start at zero; delta[h][row] is rewritten
  // for every (h, row) < (Hq, Sq) before anything reads it
  SNU1_CUDA_CHECK(cudaMemsetAsync(status, 0, sizeof(int), st));
  {
    const long long warps = (long long)Sq * Hq;
    const int blocks = (int)((warps * 32 + 255) / 256);
    attn_bwd::attn_delta_kernel<<<blocks, 256, 0, st>>>((const __nv_bfloat16*)o, ldo,
                                                        (const __nv_bfloat16*)dout, lddo, delta, Sq, Hq);
  }
  CUtensorMap tmQ, tmdO, tmK, tmV, tmQ64, tmdO64;
  if ((rc = encode_head_tmap(&tmQ, q, Sq, Hq, ldq, 128)) != kHostOk) return rc;
  if ((rc = encode_head_tmap(&tmdO, dout, Sq, Hq, lddo, 128)) != kHostOk) return rc;
  if ((rc = encode_head_tmap(&tmQ64, q, Sq, Hq, ldq, 64)) != kHostOk) return rc;
  if ((rc = encode_head_tmap(&tmdO64, dout, Sq, Hq, lddo, 64)) != kHostOk) return rc;
  if ((rc = encode_head_tmap(&tmK, k, Sk, Hkv, ldk, 128)) != kHostOk) return rc;
  if ((rc = encode_head_tmap(&tmV, v, Sk, Hkv, ldv, 128)) != kHostOk) return rc;
  attn_bwd::BwdArgs a;
  a.lse = lse;
  a.delta = delta;
  a.meta_q = (const TokMeta*)meta_q;
  a.meta_k = (const TokMeta*)meta_k;
  a.Sq = Sq;
  a.Sk = Sk;
  a.Hq = Hq;
  a.Hkv = Hkv;
  a.scale = scale;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = status;
  a.tile_slot = nullptr;  // this entry point takes no mask-bit tables: partial tiles evaluate the rule
  a.nk_tiles = nk;
  a.bits_q = nullptr;
  a.bits_k = nullptr;
  a.list = kv_list;
  a.count = kv_count;
  a.list_stride = nk;
  a.order = nullptr;
  a.out0 = (__nv_bfloat16*)dq;
  a.ld0 = lddq;
  a.out1 = nullptr;
  a.ld1 = 0;
  SNU1_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd::attn_bwd_dq_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, attn_bwd::DQ_SMEM));
  attn_bwd::attn_bwd_dq_kernel<<<dim3(Hq, nq), attn_bwd::DQ_THREADS, attn_bwd::DQ_SMEM, st>>>(
      tmQ, tmdO, tmK, tmV, a);
  a.list = q_list;
  a.count = q_count;
  a.list_stride = nq;
  a.out0 = (__nv_bfloat16*)dk;
  a.ld0 = lddk;
  a.out1 = (__nv_bfloat16*)dv;
  a.ld1 = lddv;
  SNU1_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd::attn_bwd_dkv_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, attn_bwd::DKV_SMEM));
  attn_bwd::attn_bwd_dkv_kernel<<<dim3(Hkv, nk), attn_bwd::DKV_THREADS, attn_bwd::DKV_SMEM, st>>>(
      tmQ64, tmdO64, tmK, tmV, a);
  SNU1_CUDA_CHECK(cudaGetLastError());
  if (status_out != nullptr)
    SNU1_CUDA_CHECK(cudaMemcpyAsync(status_out, status, sizeof(int), cudaMemcpyDeviceToHost, st));
  return kHostOk;
}
