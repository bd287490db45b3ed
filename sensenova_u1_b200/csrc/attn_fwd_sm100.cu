// packed_mixed_attention, forward: varlen / packed sequences, GQA, mixed
// causal-text + bidirectional-image + generation-branch gating mask, head_dim
// 128, bf16 in / fp32 softmax, for sm_100a.
//
// One CTA owns 128 query rows of one head and walks the key tiles that the
// tile classifier kept for it.  Per key tile: S = Q K^T and O += P V run on the
// tensor cores (tcgen05.mma, accumulators in TMEM: two S buffers and O), the
// four softmax warps read S with tcgen05.ld, apply the mask only on "partial"
// tiles, write P (bf16, 128-byte swizzle) to shared memory for the second
// product and rescale O in TMEM when a row maximum moved.  K and V tiles come
// through a two-stage TMA ring; V is consumed MN-major straight from its
// row-major tile.
//
// Replaces torch.compile(flex_attention) with a BlockMask in training
// (training/sensenovalm/model/modules/mha.py:35-36, 1548) and the
// flash-attn / eager attention of inference
// (src/sensenova_u1/models/neo_unify/modeling_qwen3.py:431-505, 583-745).
#include "attn_common.cuh"
#include "host_common.h"

namespace snu1 {
namespace attn {

constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int HALF_BYTES = 128 * 64 * 2;   // one 64-column box of a 128-row tile
constexpr int TILE_BYTES = 2 * HALF_BYTES;  // 32 KB
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;

// --------------------------- tile classification ---------------------------
// Besides the class of every (query tile, key tile) pair, a "partial" pair gets its mask as bits, in both
// orientations, so that the attention kernels apply it with one 16-byte load and a bit test per element
// instead of evaluating the mask rule per element (on packed multimodal batches 40 % of the kept tiles are
// partial, and the rule costs more than the softmax itself):
//   bits_q[slot][query row][4 words]   bit c of word g = query row may read key g*32 + c   (forward, dQ)
//   bits_k[slot][key row][4 words]     bit c of word g = query g*32 + c may read this key  (dK/dV)
// Slots are handed out with an atomic counter; a pair that finds the table full gets slot -1 and the
// kernels fall back to the rule for it.  Out-of-range rows and keys have zero bits.
__global__ void __launch_bounds__(128)
    classify_tiles_kernel(const TokMeta* __restrict__ mq, const TokMeta* __restrict__ mk, int Sq,
                          int Sk, unsigned char* __restrict__ cls, int nk, int* __restrict__ tile_slot,
                          uint4* __restrict__ bits_q, uint32_t* __restrict__ bits_k, int cap,
                          int* __restrict__ counter) {
  __shared__ TokMeta smk[128];
  __shared__ int s_slot;
  const int kt = blockIdx.x, qt = blockIdx.y;
  const int tid = threadIdx.x;
  const int qi = qt * 128 + tid, ki = kt * 128 + tid;
  TokMeta q, k;
  const bool q_ok = qi < Sq, k_ok = ki < Sk;
  if (q_ok) q = mq[qi];
  else q = TokMeta{-1, 0, 0, 0};
  if (k_ok) k = mk[ki];
  else k = TokMeta{-2, 0, 0, kFlagBlocked};
  smk[tid] = k;
  // quick reject on disjoint document ranges
  int qmin = q_ok ? q.doc : 0x7fffffff, qmax = q_ok ? q.doc : -0x7fffffff;
  int kmin = k_ok ? k.doc : 0x7fffffff, kmax = k_ok ? k.doc : -0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    qmin = min(qmin, __shfl_xor_sync(0xffffffffu, qmin, o));
    qmax = max(qmax, __shfl_xor_sync(0xffffffffu, qmax, o));
    kmin = min(kmin, __shfl_xor_sync(0xffffffffu, kmin, o));
    kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, o));
  }
  __shared__ int s_rng[4][4];
  if ((tid & 31) == 0) {
    s_rng[tid >> 5][0] = qmin;
    s_rng[tid >> 5][1] = qmax;
    s_rng[tid >> 5][2] = kmin;
    s_rng[tid >> 5][3] = kmax;
  }
  __syncthreads();
  qmin = min(min(s_rng[0][0], s_rng[1][0]), min(s_rng[2][0], s_rng[3][0]));
  qmax = max(max(s_rng[0][1], s_rng[1][1]), max(s_rng[2][1], s_rng[3][1]));
  kmin = min(min(s_rng[0][2], s_rng[1][2]), min(s_rng[2][2], s_rng[3][2]));
  kmax = max(max(s_rng[0][3], s_rng[1][3]), max(s_rng[2][3], s_rng[3][3]));
  if (qmax < kmin || kmax < qmin) {
    if (tid == 0) cls[(long long)qt * nk + kt] = kTileSkip;
    return;
  }
  uint32_t w[4] = {0u, 0u, 0u, 0u};
  if (q_ok) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      uint32_t ww = 0u;
#pragma unroll 8
      for (int c = 0; c < 32; ++c) ww |= (mask_allowed(q, smk[g * 32 + c]) ? 1u : 0u) << c;
      w[g] = ww;
    }
  }
  const int cnt = __popc(w[0]) + __popc(w[1]) + __popc(w[2]) + __popc(w[3]);
  const int any = __syncthreads_or(cnt > 0);
  const int all = __syncthreads_and(!q_ok || cnt == 128);
  if (tid == 0) {
    int slot = -1;
    if (any && !all && tile_slot != nullptr) {
      slot = atomicAdd(counter, 1);
      if (slot >= cap) slot = -1;
    }
    if (tile_slot != nullptr) tile_slot[(long long)qt * nk + kt] = slot;
    s_slot = slot;
    cls[(long long)qt * nk + kt] = any ? (all ? kTileFull : kTilePartial) : kTileSkip;
  }
  __syncthreads();
  const int slot = s_slot;
  if (slot < 0) return;
  bits_q[(long long)slot * 128 + tid] = make_uint4(w[0], w[1], w[2], w[3]);
  // transposed: the ballot over the 32 query rows of this warp is one word of a key's row
  const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    uint32_t keep = 0u;
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      const uint32_t b = __ballot_sync(0xffffffffu, (w[g] >> c) & 1u);
      if (lane == c) keep = b;
    }
    bits_k[((long long)slot * 128 + g * 32 + lane) * 4 + warp] = keep;
  }
}

// lists[a][..] = the b-tiles kept for a-tile a (a = query tiles when transpose == 0)
__global__ void build_lists_kernel(const unsigned char* __restrict__ cls, int nq, int nk,
                                   int transpose, int* __restrict__ lists, int* __restrict__ counts) {
  const int a = blockIdx.x * blockDim.x + threadIdx.x;
  const int na = transpose ? nk : nq, nb = transpose ? nq : nk;
  if (a >= na) return;
  int n = 0;
  for (int b = 0; b < nb; ++b) {
    const int c = transpose ? cls[(long long)b * nk + a] : cls[(long long)a * nk + b];
    if (c != kTileSkip) lists[(long long)a * nb + n++] = b | (c << 24);
  }
  counts[a] = n;
}

// lists[p][..] for the pair of query tiles (2p, 2p+1): key tiles either of them needs,
// entry = tile | classA << 24 | classB << 26
__global__ void build_pair_lists_kernel(const unsigned char* __restrict__ cls, int nq, int nk,
                                        int* __restrict__ lists, int* __restrict__ counts) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  const int np = (nq + 1) / 2;
  if (p >= np) return;
  int n = 0;
  const bool has_b = 2 * p + 1 < nq;
  for (int b = 0; b < nk; ++b) {
    const int ca = cls[(long long)(2 * p) * nk + b];
    const int cb = has_b ? cls[(long long)(2 * p + 1) * nk + b] : kTileSkip;
    if (ca != kTileSkip || cb != kTileSkip) lists[(long long)p * nk + n++] = b | (ca << 24) | (cb << 26);
  }
  counts[p] = n;
}

// --------------------------------- forward ---------------------------------
// One CTA owns TWO 128-row query tiles (A, B) of one head.  Each tile has its own
// softmax warpgroup, S accumulator, O accumulator and P buffer; they share every K / V
// tile that comes through TMA, which halves the L2 -> shared-memory traffic per FLOP and
// gives the tensor cores a second, independent stream of work while one warpgroup is in
// its exponentials.  warp 0: TMA, warp 1: MMA issue, warps 4..7: tile A, warps 8..11: tile B.
// The first warpgroup gives registers back (setmaxnreg.dec) and the softmax warpgroups take
// them (setmaxnreg.inc): a register file quarter holds three warps, so without that no warp
// could own more than 168 registers.
struct FwdArgs {
  __nv_bfloat16* O;
  long long ldo;
  float* lse;  // [Hq][Sq], log2 domain; +inf for rows without keys
  const TokMeta* meta_q;
  const TokMeta* meta_k;
  const int* pair_list;
  const int* pair_count;
  int nk;
  int Sq, Sk, Hq, Hkv;
  float scale_log2;
  int* status;
  const int* order;      // [pairs] pair indices, longest key list first; may be null
  const int* tile_slot;  // [nq][nk] slot of a partial pair's mask bits, -1 = none; may be null
  const uint4* bits_q;   // [slots][128 query rows] 128 key bits
};

constexpr int FWD_THREADS = 384;  // three warpgroups: {TMA, MMA, 2 idle}, softmax A, softmax B

__global__ void __launch_bounds__(FWD_THREADS, 1)
    attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const FwdArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;                    // 2 tiles
  uint8_t* sK = sQ + 2 * TILE_BYTES;     // 2 stages
  uint8_t* sV = sK + 2 * TILE_BYTES;     // 1 stage
  uint8_t* sP = sV + TILE_BYTES;         // 2 tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * TILE_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;
  uint64_t* v_empty = bars + 6;
  uint64_t* s_full = bars + 7;    // [2] per query tile
  uint64_t* s_empty = bars + 9;   // [2]
  uint64_t* p_full = bars + 11;   // [2]
  uint64_t* pv_done = bars + 13;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heads vary fastest, tiles follow ``order`` (most key tiles first): the CTAs with the longest lists start first
  // and the last wave holds only short ones; the query heads of one key/value head run next to each other
  const int head = blockIdx.x;
  const int pair = args.order != nullptr ? args.order[blockIdx.y] : gridDim.y - 1 - blockIdx.y;
  const int kvh = head / (args.Hq / args.Hkv);
  const int q0 = pair * 2 * BQ;
  const int n = args.pair_count[pair];
  const int* list = args.pair_list + (long long)pair * args.nk;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);
      mbar_init(&p_full[i], 4);
      mbar_init(&pv_done[i], 1);
    }
    mbar_init(v_full, 1);
    mbar_init(v_empty, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // columns: S_A [0,128) S_B [128,256) O_A [256,384) O_B [384,512)

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
  if (warp == 0) {
    if (lane == 0 && n > 0) {
      mbar_expect_tx(q_full, 2 * TILE_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        tma_load_3d(sQ + t * TILE_BYTES, &tmQ, q_full, 0, head, q0 + t * BQ);
        tma_load_3d(sQ + t * TILE_BYTES + HALF_BYTES, &tmQ, q_full, 64, head, q0 + t * BQ);
      }
      auto load_k = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&k_empty[s], ((j >> 1) & 1) ^ 1, abort_flag, args.status, 1)) return false;
        const int k0 = list_tile(list[j]) * BKV;
        mbar_expect_tx(&k_full[s], TILE_BYTES);
        tma_load_3d(sK + s * TILE_BYTES, &tmK, &k_full[s], 0, kvh, k0);
        tma_load_3d(sK + s * TILE_BYTES + HALF_BYTES, &tmK, &k_full[s], 64, kvh, k0);
        return true;
      };
      bool ok = load_k(0);
      for (int j = 0; j < n && ok; ++j) {
        if (j + 1 < n) ok = load_k(j + 1);
        if (!ok) break;
        if (!mbar_wait(v_empty, (j & 1) ^ 1, abort_flag, args.status, 1)) break;
        const int k0 = list_tile(list[j]) * BKV;
        mbar_expect_tx(v_full, TILE_BYTES);
        tma_load_3d(sV, &tmV, v_full, 0, kvh, k0);
        tma_load_3d(sV + HALF_BYTES, &tmV, v_full, 64, kvh, k0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, 128, false, true);
      bool ok = mbar_wait(q_full, 0, abort_flag, args.status, 3);
      int s_cnt[2] = {0, 0};   // S products issued per query tile
      int pv_cnt[2] = {0, 0};  // PV products issued per query tile
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        const int e = list[j];
        if (!mbar_wait(&k_full[st], (j >> 1) & 1, abort_flag, args.status, 3)) return false;
        const uint32_t k_addr = smem_u32(sK + st * TILE_BYTES);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (((e >> (24 + 2 * t)) & 3) == kTileSkip) continue;
          // the softmax warpgroup must have drained the previous S of this tile
          if (!mbar_wait(&s_empty[t], (s_cnt[t] & 1) ^ 1, abort_flag, args.status, 2)) return false;
          tc_fence_after();
          const uint32_t q_addr = smem_u32(sQ + t * TILE_BYTES);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
            umma_bf16_ss(tmem_base + t * 128, make_smem_desc(q_addr + off, 0, 1024),
                         make_smem_desc(k_addr + off, 0, 1024), idesc_s, k > 0 ? 1u : 0u);
          }
          umma_commit(&s_full[t]);
          ++s_cnt[t];
        }
        umma_commit(&k_empty[st]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n && ok; ++j) {
        if (j + 1 < n) {
          ok = issue_s(j + 1);
          if (!ok) break;
        }
        const int e = list[j];
        if (!mbar_wait(v_full, j & 1, abort_flag, args.status, 3)) {
          ok = false;
          break;
        }
        const uint32_t v_addr = smem_u32(sV);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (((e >> (24 + 2 * t)) & 3) == kTileSkip) continue;
          if (!mbar_wait(&p_full[t], pv_cnt[t] & 1, abort_flag, args.status, 2)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t p_addr = smem_u32(sP + t * TILE_BYTES);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t a_off = (k >> 2) * HALF_BYTES + (k & 3) * 32;
            umma_bf16_ss(tmem_base + 256 + t * 128, make_smem_desc(p_addr + a_off, 0, 1024),
                         make_smem_desc(v_addr + k * 2048, HALF_BYTES, 1024), idesc_pv,
                         (pv_cnt[t] > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&pv_done[t]);
          ++pv_cnt[t];
        }
        if (!ok) break;
        umma_commit(v_empty);
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    // ------------------------------ softmax --------------------------------
    const int t = (warp - 4) >> 2;   // query tile of this warpgroup
    const int quarter = warp & 3;
    const int rloc = quarter * 32 + lane;  // TMEM lane == row in the tile
    const int row = q0 + t * BQ + rloc;
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    const uint32_t tmem_S = tmem_base + t * 128;
    const uint32_t tmem_O = tmem_base + 256 + t * 128;
    uint8_t* sPt = sP + t * TILE_BYTES;
    TokMeta mq = row < args.Sq ? args.meta_q[row] : TokMeta{-1, 0, 0, 0};
    float m = -INFINITY, l = 0.f;
    const float sc = args.scale_log2;
    bool ok = true;
    int cnt = 0;  // key tiles this query tile has processed
    for (int j = 0; j < n && ok; ++j) {
      const int entry = list[j];
      const int cls_t = (entry >> (24 + 2 * t)) & 3;
      if (cls_t == kTileSkip) continue;
      const bool partial = cls_t != kTileFull;
      const int k0 = list_tile(entry) * BKV;
      if (!mbar_wait(&s_full[t], cnt & 1, abort_flag, args.status, 5)) {
        ok = false;
        break;
      }
      tc_fence_after();
      float sv[128];
      {
        uint32_t r0[32], r1[32], r2[32], r3[32];
        const uint32_t ta = tmem_S + lane_sel;
        tmem_ld_32x32b_x32(ta, r0);
        tmem_ld_32x32b_x32(ta + 32, r1);
        tmem_ld_32x32b_x32(ta + 64, r2);
        tmem_ld_32x32b_x32(ta + 96, r3);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          sv[c] = __uint_as_float(r0[c]);
          sv[32 + c] = __uint_as_float(r1[c]);
          sv[64 + c] = __uint_as_float(r2[c]);
          sv[96 + c] = __uint_as_float(r3[c]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[t]);
      if (partial) {
        uint32_t w[4];
        const int slot =
            args.tile_slot != nullptr ? __ldg(args.tile_slot + (long long)(2 * pair + t) * args.nk + list_tile(entry)) : -1;
        if (slot >= 0) {
          const uint4 u = __ldg(args.bits_q + (long long)slot * 128 + rloc);
          w[0] = u.x;
          w[1] = u.y;
          w[2] = u.z;
          w[3] = u.w;
        } else {
          mask_words_by_rule<4>(mq, args.meta_k + k0, args.Sk - k0, true, w);
        }
        // Left of a causal diagonal (and inside an image block) a 32-key word is all ones for every row of the warp:
        // no per-element test there.
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          if (__all_sync(0xffffffffu, w[g] == 0xffffffffu)) continue;
#pragma unroll
          for (int c = 0; c < 32; ++c)
            if (!((w[g] >> c) & 1u)) sv[g * 32 + c] = -INFINITY;
        }
      }
      // row maximum: four independent chains of 3-input max (a single chain of 127 dependent
      // operations left the scheduler with nothing to issue)
      float mx;
      {
        float m0 = sv[0], m1 = sv[1], m2 = sv[2], m3 = sv[3];
#pragma unroll
        for (int c = 4; c < 124; c += 8) {
          m0 = max3(m0, sv[c], sv[c + 1]);
          m1 = max3(m1, sv[c + 2], sv[c + 3]);
          m2 = max3(m2, sv[c + 4], sv[c + 5]);
          m3 = max3(m3, sv[c + 6], sv[c + 7]);
        }
        m0 = max3(m0, sv[124], sv[125]);
        m1 = max3(m1, sv[126], sv[127]);
        mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      }
      // Lazy rescaling: the running maximum only moves when some row of the warp outgrows it by more
      // than 2^8 (in the exponent domain); until then the exponentials are taken against the stale
      // maximum (values up to 256, exact enough in fp32 / bf16) and the accumulator O is left alone.
      const bool grow = mx * sc > m * sc + 8.f;      // also true for the first finite maximum (m = -inf)
      const bool rescale = __any_sync(0xffffffffu, grow);
      const float m_new = rescale ? fmaxf(m, mx) : m;
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = rescale ? fast_exp2((m - m_use) * sc) : 1.f;
      const float mb = m_use * sc;
      float sum;
      {
        const uint64_t sc2 = pack_f32x2(sc, sc), nb2 = pack_f32x2(-mb, -mb);
        uint64_t a0 = pack_f32x2(0.f, 0.f), a1 = a0, a2 = a0, a3 = a0;
#pragma unroll
        for (int c = 0; c < 128; c += 8) {
          uint64_t t0 = fma_f32x2(pack_f32x2(sv[c], sv[c + 1]), sc2, nb2);
          uint64_t t1 = fma_f32x2(pack_f32x2(sv[c + 2], sv[c + 3]), sc2, nb2);
          uint64_t t2 = fma_f32x2(pack_f32x2(sv[c + 4], sv[c + 5]), sc2, nb2);
          uint64_t t3 = fma_f32x2(pack_f32x2(sv[c + 6], sv[c + 7]), sc2, nb2);
          float x0, x1, x2, x3, x4, x5, x6, x7;
          unpack_f32x2(t0, x0, x1);
          unpack_f32x2(t1, x2, x3);
          unpack_f32x2(t2, x4, x5);
          unpack_f32x2(t3, x6, x7);
          sv[c] = fast_exp2(x0);
          sv[c + 1] = fast_exp2(x1);
          sv[c + 2] = fast_exp2(x2);
          sv[c + 3] = fast_exp2(x3);
          sv[c + 4] = fast_exp2(x4);
          sv[c + 5] = fast_exp2(x5);
          sv[c + 6] = fast_exp2(x6);
          sv[c + 7] = fast_exp2(x7);
          a0 = add_f32x2(a0, pack_f32x2(sv[c], sv[c + 1]));
          a1 = add_f32x2(a1, pack_f32x2(sv[c + 2], sv[c + 3]));
          a2 = add_f32x2(a2, pack_f32x2(sv[c + 4], sv[c + 5]));
          a3 = add_f32x2(a3, pack_f32x2(sv[c + 6], sv[c + 7]));
        }
        float s0, s1;
        unpack_f32x2(add_f32x2(add_f32x2(a0, a1), add_f32x2(a2, a3)), s0, s1);
        sum = s0 + s1;
      }
      l = l * alpha + sum;
      m = m_new;
      if (cnt > 0) {
        if (!mbar_wait(&pv_done[t], (cnt - 1) & 1, abort_flag, args.status, 5)) {
          ok = false;
          break;
        }
        tc_fence_after();
      }
#pragma unroll
      for (int ch = 0; ch < 16; ++ch) {
        uint4 u;
        u.x = pack_bf16x2(sv[ch * 8 + 0], sv[ch * 8 + 1]);
        u.y = pack_bf16x2(sv[ch * 8 + 2], sv[ch * 8 + 3]);
        u.z = pack_bf16x2(sv[ch * 8 + 4], sv[ch * 8 + 5]);
        u.w = pack_bf16x2(sv[ch * 8 + 6], sv[ch * 8 + 7]);
        *reinterpret_cast<uint4*>(sPt + (ch >> 3) * HALF_BYTES + swz128_offset(rloc, ch & 7)) = u;
      }
      if (cnt > 0 && rescale) {
        const uint64_t al2 = pack_f32x2(alpha, alpha);
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_O + c * 32 + lane_sel, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float y0, y1;
            unpack_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), al2), y0, y1);
            r[i] = __float_as_uint(y0);
            r[i + 1] = __float_as_uint(y1);
          }
          tmem_st_32x32b_x32(tmem_O + c * 32 + lane_sel, r);
        }
        tmem_st_wait();
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
      ++cnt;
    }
    if (cnt == 0) {
      // no key tile at all for this query tile: zero output
      if (ok && row < args.Sq) {
        uint4 z = make_uint4(0, 0, 0, 0);
        uint4* op = reinterpret_cast<uint4*>(args.O + (long long)row * args.ldo + head * 128);
#pragma unroll
        for (int i = 0; i < 16; ++i) op[i] = z;
        args.lse[(long long)head * args.Sq + row] = __int_as_float(0x7f800000);
      }
    } else if (ok && mbar_wait(&pv_done[t], (cnt - 1) & 1, abort_flag, args.status, 5)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_O + c * 32 + lane_sel, r);
        tmem_ld_wait();
        if (row < args.Sq) {
          uint4* op = reinterpret_cast<uint4*>(args.O + (long long)row * args.ldo + head * 128 + c * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(r[i * 8 + 0]) * inv, __uint_as_float(r[i * 8 + 1]) * inv);
            u.y = pack_bf16x2(__uint_as_float(r[i * 8 + 2]) * inv, __uint_as_float(r[i * 8 + 3]) * inv);
            u.z = pack_bf16x2(__uint_as_float(r[i * 8 + 4]) * inv, __uint_as_float(r[i * 8 + 5]) * inv);
            u.w = pack_bf16x2(__uint_as_float(r[i * 8 + 6]) * inv, __uint_as_float(r[i * 8 + 7]) * inv);
            op[i] = u;
          }
        }
        __syncwarp();
      }
      if (row < args.Sq)
        args.lse[(long long)head * args.Sq + row] =
            l > 0.f ? (m * sc + log2f(l)) : __int_as_float(0x7f800000);
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

constexpr int FWD_SMEM = 7 * TILE_BYTES + 256 + 1024;

}  // namespace attn

// rows x heads x 128 view of a strided bf16 tensor; box = 128 rows x 1 head x 64 dims
int encode_head_tmap(CUtensorMap* out, const void* base, long long rows, int heads, long long ld,
                     int box_rows) {
  uint64_t dims[3] = {128, (uint64_t)heads, (uint64_t)rows};
  uint64_t strides[2] = {128 * 2, (uint64_t)ld * 2};
  uint32_t box[3] = {64, 1, (uint32_t)box_rows};
  return encode_tmap_bf16(out, base, 3, dims, strides, box);
}

}  // namespace snu1

using namespace snu1;

// cls: [nq][nk] bytes; kv_list: [nq][nk] ints; kv_count: [nq]; q_list: [nk][nq]; q_count: [nk];
// pair_list: [ceil(nq/2)][nk]; pair_count: [ceil(nq/2)].
// tile_slot: [nq][nk] ints; bits_q / bits_k: [cap][128][4] words each; counter: one int (zeroed here).
// tile_slot may be null (no mask bits: the kernels evaluate the rule on partial tiles).
SNU1_API int snu1_attn_build_tiles(const void* meta_q, const void* meta_k, int Sq, int Sk,
                                   unsigned char* cls, int* kv_list, int* kv_count, int* q_list,
                                   int* q_count, int* pair_list, int* pair_count, int* tile_slot,
                                   void* bits_q, void* bits_k, int cap, int* counter, void* stream) {
  if (Sq <= 0 || Sk <= 0) {
    set_last_error("attn_build_tiles: empty sequence");
    return kHostBadArg;
  }
  const int nq = (Sq + 127) / 128, nk = (Sk + 127) / 128;
  cudaStream_t st = (cudaStream_t)stream;
  if (tile_slot != nullptr) {
    if (bits_q == nullptr || bits_k == nullptr || counter == nullptr || cap < 0) {
      set_last_error("attn_build_tiles: mask-bit tables missing");
      return kHostBadArg;
    }
    SNU1_CUDA_CHECK(cudaMemsetAsync(counter, 0, sizeof(int), st));
  }
  attn::classify_tiles_kernel<<<dim3(nk, nq), 128, 0, st>>>((const TokMeta*)meta_q, (const TokMeta*)meta_k, Sq, Sk,
                                                            cls, nk, tile_slot, (uint4*)bits_q, (uint32_t*)bits_k,
                                                            cap, counter);
  attn::build_lists_kernel<<<(nq + 63) / 64, 64, 0, st>>>(cls, nq, nk, 0, kv_list, kv_count);
  if (q_list != nullptr)
    attn::build_lists_kernel<<<(nk + 63) / 64, 64, 0, st>>>(cls, nq, nk, 1, q_list, q_count);
  attn::build_pair_lists_kernel<<<((nq + 1) / 2 + 63) / 64, 64, 0, st>>>(cls, nq, nk, pair_list, pair_count);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_attn_fwd(const void* q, long long ldq, const void* k, long long ldk, const void* v,
                           long long ldv, void* o, long long ldo, float* lse, const void* meta_q,
                           const void* meta_k, const int* pair_list, const int* pair_count, int Sq,
                           int Sk, int Hq, int Hkv, float scale, const int* tile_slot, const void* bits_q,
                           const int* pair_order, void* stream) {
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || Sq <= 0 || Sk <= 0) {
    set_last_error("attn_fwd: bad head counts / lengths");
    return kHostBadArg;
  }
  if (ldq % 8 || ldk % 8 || ldv % 8 || ldo % 8) {
    set_last_error("attn_fwd: row strides must be multiples of 8 elements");
    return kHostBadArg;
  }
  CUtensorMap tmQ, tmK, tmV;
  int rc;
  if ((rc = encode_head_tmap(&tmQ, q, Sq, Hq, ldq, 128)) != kHostOk) return rc;
  if ((rc = encode_head_tmap(&tmK, k, Sk, Hkv, ldk, 128)) != kHostOk) return rc;
  if ((rc = encode_head_tmap(&tmV, v, Sk, Hkv, ldv, 128)) != kHostOk) return rc;
  attn::FwdArgs a;
  a.O = (__nv_bfloat16*)o;
  a.ldo = ldo;
  a.lse = lse;
  a.meta_q = (const TokMeta*)meta_q;
  a.meta_k = (const TokMeta*)meta_k;
  a.pair_list = pair_list;
  a.pair_count = pair_count;
  a.nk = (Sk + 127) / 128;
  a.Sq = Sq;
  a.Sk = Sk;
  a.Hq = Hq;
  a.Hkv = Hkv;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.status = device_status_word();
  a.tile_slot = bits_q != nullptr ? tile_slot : nullptr;
  a.bits_q = (const uint4*)bits_q;
  a.order = pair_order;
  const int nq = (Sq + 127) / 128;
  SNU1_CUDA_CHECK(cudaFuncSetAttribute(attn::attn_fwd_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, attn::FWD_SMEM));
  attn::attn_fwd_kernel<<<dim3(Hq, (nq + 1) / 2), attn::FWD_THREADS, attn::FWD_SMEM, (cudaStream_t)stream>>>(
      tmQ, tmK, tmV, a);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}
