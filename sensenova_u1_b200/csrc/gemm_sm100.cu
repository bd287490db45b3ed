// mot_gemm: persistent, warp-specialised bf16 GEMM for sm_100a.
//
//   * operands arrive in shared memory through TMA (cp.async.bulk.tensor,
//     128-byte swizzle, 4-stage mbarrier ring, no multicast);
//   * the product is issued by one elected thread as tcgen05.mma
//     (cta_group::1, 128x256x16 per instruction) with fp32 accumulators in TMEM;
//   * two 256-column accumulators (all 512 TMEM columns) let the epilogue warps
//     drain tile i with tcgen05.ld while the tensor cores already work on i+1;
//   * one CTA per SM, static tile schedule banded over M for L2 reuse.
//
// Two kernels share this structure.  Products without a fused collective run on
// the pair kernel (mot_gemm_pair_kernel: clusters of two CTAs, tcgen05.mma
// cta_group::2 on 256x256 tiles, six 32 KB stages per CTA); the single-CTA kernel
// (mot_gemm_kernel, 128x256 tiles) carries the fused all-gather and reduce-scatter
// forms and stays selectable for everything (snu1_gemm_set_pair_mode).
//
// Both operands may be K-major or MN-major, so that the forward product
// (x W^T), the data gradient (dy W) and the weight gradient (dy^T x) all run
// on the row-major tensors as they are, with no transposed copies.
//
// Grouping (one launch for all modality branches / experts):
//   group_mode 1: the rows of A are partitioned in 128-row tiles; tile t uses
//                 weight set tile_group[t] (device array, -1 = skip the tile).
//                 This is the MoT "generation rows | understanding rows" split
//                 (reference: training/sensenovalm/model/modeling_qwen3_moe_mot.py:323-369
//                 does it with slices and torch.cat) and the MoE expert split
//                 (reference: training/sensenovalm/model/ops/linear.py:167-187).
//   group_mode 2: weight gradients; output g reduces over the row range
//                 [k_begin[g], k_end[g]) of both operands (device arrays).
//
// Replaces the cuBLAS / fused_dense call sites of the reference
// (training/sensenovalm/model/ops/linear.py:108-165).
#include <string.h>

#include "host_common.h"
#include "sm100_common.cuh"

namespace snu1 {

namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int MN_CHUNK_BYTES = 64 * BK * 2;  // one 64-wide MN-major box: 8 KB
constexpr int NUM_THREADS = 192;             // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int BAND = 16;  // M tiles per scheduling band

struct Args {
  int M, N, K;
  int group_mode;
  int num_groups;
  const int* tile_group;
  const int* k_begin;
  const int* k_end;
  void* C;
  long long ldc;
  long long c_group_stride;
  const int* m_rows_dev;  // optional: number of rows of A / C in use (device scalar), <= M
  int pair_band;          // pair kernel: 256-row pair tiles per scheduling band
  int out_mode;  // 0 bf16 store, 1 bf16 accumulate, 2 fp32 store, 3 fp32 accumulate
  const __nv_bfloat16* residual;
  long long ldr;
  float alpha;
  int* status;
  // ---- fused all-gather of operand B's rows (weight shards living on peer GPUs) ----
  // The first `num_copy_ctas` CTAs pull every rank's shard [shard_rows][K] through shared memory
  // (1-D bulk TMA, no multicast) into the local staging buffer that tmB describes and publish one
  // flag per `chunk_rows` rows; the GEMM CTAs walk the shards in ring order starting with the local
  // one and wait (bounded) for a chunk's flag before they load from it.
  int gather_b;              // 0: off
  int num_copy_ctas;
  int world, my_rank;
  const void* shard[8];      // peer pointers of the row shards (K-major rows)
  void* staging;             // [world * shard_rows][K] local
  int shard_rows, chunk_rows;
  long long row_bytes;
  int* gather_flags;         // [world * shard_rows / chunk_rows], compared against gather_seq
  int gather_seq;
  // ---- fused reduce-scatter epilogue (out_mode 4): rows of C are owned by ranks in blocks of
  // rs_rows; the tile is added (fp32 red) into the owner's buffer through its peer pointer ----
  float* rs_dst[8];
  int rs_rows;
};

struct TileCoord {
  int m_tile, n_tile, group;
  int k_lo, k_hi;  // reduction range in elements
  bool skip;
};

__device__ __forceinline__ TileCoord decode_tile(const Args& a, int t, int num_m, int num_n) {
  TileCoord c;
  int per_group = num_m * num_n;
  int g = 0;
  if (a.group_mode == 2) {
    g = t / per_group;
    t -= g * per_group;
  }
  int n_base = 0, nn = num_n;
  if (a.gather_b) {
    // all tiles of one shard before the next shard, local shard first
    const int n_per_shard = num_n / a.world;
    const int per_shard = num_m * n_per_shard;
    const int step = t / per_shard;
    t -= step * per_shard;
    n_base = ((a.my_rank + step) % a.world) * n_per_shard;
    nn = n_per_shard;
  }
  int band_tiles = BAND * nn;
  int band = t / band_tiles;
  int within = t - band * band_tiles;
  int rows = min(BAND, num_m - band * BAND);
  c.n_tile = within / rows;
  c.m_tile = band * BAND + (within - c.n_tile * rows);
  c.n_tile += n_base;
  c.skip = false;
  c.k_lo = 0;
  c.k_hi = a.K;
  c.group = 0;
  if (a.group_mode == 1) {
    int tg = a.tile_group[c.m_tile];
    c.skip = tg < 0 || tg >= a.num_groups;
    c.group = c.skip ? 0 : tg;
  } else if (a.group_mode == 2) {
    c.group = g;
    c.k_lo = a.k_begin[g];
    c.k_hi = min(a.k_end[g], a.K);
    if (c.k_hi < c.k_lo) c.k_hi = c.k_lo;
  }
  return c;
}


__device__ __forceinline__ void red_add_v4_f32(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// bounded spin on a flag written by another CTA of this kernel
__device__ __forceinline__ bool wait_flag_gpu(const int* f, int want, volatile int* abort_flag, int* status) {
  if (ld_acquire_gpu(f) >= want) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (ld_acquire_gpu(f) < want) {
    if ((++spins & 0xff) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > kPeerWaitNs) {
        *abort_flag = 1;
        report_status(status, kPeerTimeout, 7);
        return false;
      }
    }
  }
  return true;
}
// 1-D bulk copies (TMA engine, no tensor map, no multicast)
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// Copy role of the fused all-gather: one thread drives the TMA engine.  Work item = one chunk of one
// rank's shard; items are dealt round-robin to the copy CTAs in ring order (local shard first), each
// moved through a 4-slot ring of 32 KB shared-memory pieces.
constexpr int COPY_PIECE = 32768;
constexpr int COPY_SLOTS = 4;
__device__ void gather_copy_cta(const Args& a, uint8_t* smem, uint64_t* bars) {
  if (threadIdx.x != 0) return;
  for (int i = 0; i < COPY_SLOTS; ++i) mbar_init(&bars[i], 1);
  mbar_fence_init();
  const int chunks_per_shard = a.shard_rows / a.chunk_rows;
  const long long chunk_bytes = (long long)a.chunk_rows * a.row_bytes;
  const int items = (a.world - 1) * chunks_per_shard;   // the local shard is read in place
  uint32_t use[COPY_SLOTS] = {0, 0, 0, 0};   // completed loads per slot (phase tracking)
  uint32_t piece_idx = 0;
  for (int w = blockIdx.x; w < items; w += a.num_copy_ctas) {
    const int step = 1 + w / chunks_per_shard, ch = w % chunks_per_shard;
    const int src_rank = (a.my_rank + step) % a.world;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(a.shard[src_rank]) + (long long)ch * chunk_bytes;
    uint8_t* dst = reinterpret_cast<uint8_t*>(a.staging) +
                   ((long long)src_rank * chunks_per_shard + ch) * chunk_bytes;
    // software pipeline: COPY_SLOTS - 1 loads in flight, each piece stored once it landed.  Piece i reuses the
    // slot of piece i - COPY_SLOTS, whose store is store group i - COPY_SLOTS.  With at most COPY_SLOTS - 1
    // pieces issued beyond the stored ones, stores 0 .. i - COPY_SLOTS + 1 are committed when piece i is issued,
    // so "at most one store group still reading" means every group up to i - COPY_SLOTS has released its slot.
    const long long npieces = (chunk_bytes + COPY_PIECE - 1) / COPY_PIECE;
    long long issued = 0, stored = 0;
    uint32_t first_piece = piece_idx;
    while (stored < npieces) {
      while (issued < npieces && issued - stored < COPY_SLOTS - 1) {
        const int slot = (first_piece + issued) % COPY_SLOTS;
        bulk_wait_read<1>();
        const long long off = issued * COPY_PIECE;
        const uint32_t bytes = (uint32_t)min((long long)COPY_PIECE, chunk_bytes - off);
        mbar_expect_tx(&bars[slot], bytes);
        bulk_g2s(smem + slot * COPY_PIECE, src + off, bytes, &bars[slot]);
        ++issued;
      }
      const int slot = (first_piece + stored) % COPY_SLOTS;
      volatile int dummy_abort = 0;
      if (!mbar_wait(&bars[slot], use[slot] & 1, &dummy_abort, a.status, 1)) return;
      ++use[slot];
      const long long off = stored * COPY_PIECE;
      const uint32_t bytes = (uint32_t)min((long long)COPY_PIECE, chunk_bytes - off);
      fence_proxy_async_all();
      bulk_s2g(dst + off, smem + slot * COPY_PIECE, bytes);
      bulk_commit();
      ++stored;
    }
    piece_idx = first_piece + (uint32_t)npieces;
    bulk_wait_all<0>();          // the chunk is in local memory
    fence_proxy_async_all();
    __threadfence();
    st_release_gpu(a.gather_flags + src_rank * chunks_per_shard + ch, a.gather_seq);
  }
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    mot_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmBlocal, const Args args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full_bar = bars;                  // [STAGES]
  uint64_t* empty_bar = bars + STAGES;        // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES;     // [2]
  uint64_t* acc_empty = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // rows in use (optional device scalar): buffers sized for a worst case are walked only up to their fill,
  // instead of decoding and skipping thousands of empty row tiles
  int m_eff = args.M;
  if (args.m_rows_dev != nullptr) m_eff = min(m_eff, max(*args.m_rows_dev, 0));
  const int num_m = (m_eff + BM - 1) / BM;
  const int num_n = (args.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n * (args.group_mode == 2 ? args.num_groups : 1);
  const int ncopy = args.gather_b ? args.num_copy_ctas : 0;

  if ((int)blockIdx.x < ncopy) {
    gather_copy_cta(args, smem, reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES));
    return;
  }
  const int cta = blockIdx.x - ncopy;         // index among the GEMM CTAs
  const int ncta = gridDim.x - ncopy;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += ncta) {
        TileCoord tc = decode_tile(args, t, num_m, num_n);
        if (tc.skip) continue;
        const int m0 = tc.m_tile * BM;
        const int n0 = tc.n_tile * BN;
        bool gather_ready = false;
        for (int k0 = tc.k_lo; k0 < tc.k_hi; k0 += BK, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, args.status, 1)) {
            ok = false;
            break;
          }
          const bool b_local = args.gather_b && (n0 / args.shard_rows) == args.my_rank;
          if (args.gather_b && !gather_ready && !b_local) {
            // the 256 B rows of this tile sit in chunks [n0 / chunk_rows, (n0 + 255) / chunk_rows]
            const int c0 = n0 / args.chunk_rows, c1 = min(n0 + BN - 1, args.N - 1) / args.chunk_rows;
            for (int c = c0; c <= c1 && ok; ++c) ok = wait_flag_gpu(args.gather_flags + c, args.gather_seq, abort_flag, args.status);
            if (!ok) break;
            fence_proxy_async_all();
            gather_ready = true;
          }
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          uint8_t* a_dst = sA + s * A_STAGE_BYTES;
          uint8_t* b_dst = sB + s * B_STAGE_BYTES;
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i)
              tma_load_2d(a_dst + i * MN_CHUNK_BYTES, &tmA, &full_bar[s], m0 + 64 * i, k0);
          } else {
            tma_load_2d(a_dst, &tmA, &full_bar[s], k0, m0);
          }
          if (B_MN) {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              tma_load_3d(b_dst + i * MN_CHUNK_BYTES, &tmB, &full_bar[s], n0 + 64 * i, k0,
                          args.group_mode == 1 ? tc.group : 0);
          } else if (b_local) {
            // this rank's own rows: straight from the shard, no staging copy and no flag
            tma_load_3d(b_dst, &tmBlocal, &full_bar[s], k0, n0 - args.my_rank * args.shard_rows, 0);
          } else {
            tma_load_3d(b_dst, &tmB, &full_bar[s], k0, n0, args.group_mode == 1 ? tc.group : 0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      uint32_t it = 0;
      uint32_t tile_it = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += ncta) {
        TileCoord tc = decode_tile(args, t, num_m, num_n);
        if (tc.skip) continue;
        const int acc = tile_it & 1;
        const uint32_t acc_ph = (tile_it >> 1) & 1;
        if (!mbar_wait(&acc_empty[acc], acc_ph ^ 1, abort_flag, args.status, 2)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool first = true;
        for (int k0 = tc.k_lo; k0 < tc.k_hi; k0 += BK, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, args.status, 3)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(sA + s * A_STAGE_BYTES);
          const uint32_t b_addr = smem_u32(sB + s * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN ? make_smem_desc(a_addr + k * (UMMA_K * 128), MN_CHUNK_BYTES, 1024)
                                     : make_smem_desc(a_addr + k * (UMMA_K * 2), 0, 1024);
            const uint64_t db = B_MN ? make_smem_desc(b_addr + k * (UMMA_K * 128), MN_CHUNK_BYTES, 1024)
                                     : make_smem_desc(b_addr + k * (UMMA_K * 2), 0, 1024);
            umma_bf16_ss(d_tmem, da, db, idesc, first ? 0u : 1u);
            first = false;
          }
          umma_commit(&empty_bar[s]);  // smem stage reusable once these MMAs retire
        }
        if (!ok) break;
        umma_commit(&acc_full[acc]);
        ++tile_it;
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32)
    uint32_t tile_it = 0;
    bool ok = true;
    for (int t = cta; t < num_tiles && ok; t += ncta) {
      TileCoord tc = decode_tile(args, t, num_m, num_n);
      if (tc.skip) continue;
      const int acc = tile_it & 1;
      const uint32_t acc_ph = (tile_it >> 1) & 1;
      if (!mbar_wait(&acc_full[acc], acc_ph, abort_flag, args.status, 4)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const bool has_acc = tc.k_hi > tc.k_lo;
      const int row = tc.m_tile * BM + quarter * 32 + lane;
      const bool row_ok = row < args.M;
      const int n0 = tc.n_tile * BN;
      const long long c_off =
          (args.group_mode == 2 ? tc.group * args.c_group_stride : 0) + (long long)row * args.ldc;
#pragma unroll 1
      for (int ch = 0; ch < BN / 32; ++ch) {
        const int col0 = n0 + ch * 32;
        if (col0 >= args.N) break;  // warp-uniform
        uint32_t r[32];
        if (has_acc) {
          tmem_ld_32x32b_x32(tmem_base + acc * BN + ch * 32 + ((uint32_t)(quarter * 32) << 16), r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
        __syncwarp();
        if (row_ok) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * args.alpha;
        const int ncols = min(32, args.N - col0);  // multiple of 8 (host checks N % 8 == 0)
        if (args.out_mode <= 1) {
          __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(args.C) + c_off + col0;
          const __nv_bfloat16* rp =
              args.residual ? args.residual + (long long)row * args.ldr + col0 : nullptr;
#pragma unroll
          for (int j8 = 0; j8 < 4; ++j8) {
            if (j8 * 8 >= ncols) break;
            if (args.out_mode == 1) {
              uint4 old = *reinterpret_cast<const uint4*>(cp + j8 * 8);
              const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                float2 f = __bfloat1622float2(o2[q]);
                v[j8 * 8 + 2 * q] += f.x;
                v[j8 * 8 + 2 * q + 1] += f.y;
              }
            }
            if (rp) {
              uint4 rr = *reinterpret_cast<const uint4*>(rp + j8 * 8);
              const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rr);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                float2 f = __bfloat1622float2(r2[q]);
                v[j8 * 8 + 2 * q] += f.x;
                v[j8 * 8 + 2 * q + 1] += f.y;
              }
            }
            uint4 o;
            o.x = pack_bf16x2(v[j8 * 8 + 0], v[j8 * 8 + 1]);
            o.y = pack_bf16x2(v[j8 * 8 + 2], v[j8 * 8 + 3]);
            o.z = pack_bf16x2(v[j8 * 8 + 4], v[j8 * 8 + 5]);
            o.w = pack_bf16x2(v[j8 * 8 + 6], v[j8 * 8 + 7]);
            *reinterpret_cast<uint4*>(cp + j8 * 8) = o;
          }
        } else if (args.out_mode == 5) {
          // reduce-scatter, staged form: this rank's bf16 partial rows go to ITS slab of the owner's staging
          // buffer ([world][rs_rows][ldc] bf16 on every rank) with plain 16-byte peer stores; the owner sums
          // the slabs afterwards.  Half the NVLink bytes of the fp32 form and no atomics.
          const int owner = row / args.rs_rows;
          __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(args.rs_dst[owner]) +
                              ((long long)args.my_rank * args.rs_rows + (row - owner * args.rs_rows)) * args.ldc + col0;
#pragma unroll
          for (int j8 = 0; j8 < 4; ++j8) {
            if (j8 * 8 >= ncols) break;
            uint4 o;
            o.x = pack_bf16x2(v[j8 * 8 + 0], v[j8 * 8 + 1]);
            o.y = pack_bf16x2(v[j8 * 8 + 2], v[j8 * 8 + 3]);
            o.z = pack_bf16x2(v[j8 * 8 + 4], v[j8 * 8 + 5]);
            o.w = pack_bf16x2(v[j8 * 8 + 6], v[j8 * 8 + 7]);
            *reinterpret_cast<uint4*>(cp + j8 * 8) = o;
          }
        } else if (args.out_mode == 4) {
          // reduce-scatter: fp32 red into the buffer of the rank that owns this row
          const int owner = row / args.rs_rows;
          float* cp = args.rs_dst[owner] + (long long)(row - owner * args.rs_rows) * args.ldc + col0;
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            if (j4 * 4 >= ncols) break;
            red_add_v4_f32(cp + j4 * 4, v[j4 * 4], v[j4 * 4 + 1], v[j4 * 4 + 2], v[j4 * 4 + 3]);
          }
        } else {
          float* cp = reinterpret_cast<float*>(args.C) + c_off + col0;
#pragma unroll
          for (int j4 = 0; j4 < 8; ++j4) {
            if (j4 * 4 >= ncols) break;
            float4 o = make_float4(v[j4 * 4], v[j4 * 4 + 1], v[j4 * 4 + 2], v[j4 * 4 + 3]);
            if (args.out_mode == 3) {
              float4 old = *reinterpret_cast<const float4*>(cp + j4 * 4);
              o.x += old.x;
              o.y += old.y;
              o.z += old.z;
              o.w += old.w;
            }
            *reinterpret_cast<float4*>(cp + j4 * 4) = o;
          }
        }
        }  // row_ok
        __syncwarp();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      ++tile_it;
    }
  }

  // ------------------------------ teardown ------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag) {
      // give copies and MMAs still in flight a bounded time to land before the
      // shared memory and TMEM of this CTA are handed back
      uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 2000000ull) {
      }
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}


// =====================================================================================
// Pair kernel: two CTAs of a cluster (two SMs) work on one 256x256 output tile with
// tcgen05.mma.cta_group::2.  CTA r of the pair holds rows [128 r, 128 r + 128) of the A
// tile and columns [128 r, 128 r + 128) of the B tile in ITS shared memory and the
// accumulator rows [128 r, 128 r + 128) in ITS tensor memory, so every SM feeds its
// tensor core 8 KB of operands per 128x256x16 product instead of 12 KB, and six stages of
// 32 KB fit where four of 48 KB did.  The even CTA issues all products; TMA loads of both
// CTAs complete on the even CTA's "full" barriers (cta_group::2 form, no multicast);
// "stage free" and "accumulator ready" reach both CTAs by one tcgen05.commit each;
// "accumulator drained" comes back to the even CTA by remote mbarrier arrives.
//
// group_mode 1 with a pair of row tiles that belong to different weight sets runs the
// pair once per set, each time storing only the half that belongs to it.
// =====================================================================================
constexpr int P_STAGES = 6;
constexpr int P_BN_HALF = 128;
constexpr int P_A_BYTES = BM * BK * 2;         // 16 KB: this CTA's 128 rows of A
constexpr int P_B_BYTES = P_BN_HALF * BK * 2;  // 16 KB: this CTA's 128 columns of B
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + 1024 + 256;
constexpr int P_BAND = 8;                      // pair rows (256 rows each) per scheduling band

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cl(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// bounded wait, cluster-scope acquire (the arrival may come from the other CTA of the pair)
__device__ __forceinline__ bool mbar_wait_cl(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status,
                                             int where) {
  if (mbar_try_wait_cl(bar, parity)) return true;
  uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (!mbar_try_wait_cl(bar, parity)) {
    if ((++spins & 0x3ff) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > kLocalWaitNs) {
        *abort_flag = 1;
        report_status(status, kWaitTimeout, where);
        return false;
      }
    }
  }
  return true;
}
// TMA loads whose completion is counted on a barrier of the pair's even CTA (no multicast)
__device__ __forceinline__ void tma_pair_load_2d(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_pair_load_3d(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr,
                                                 int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_pair_bf16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                  uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on the barrier at `cluster_addr` (either CTA of the pair) once all earlier products have retired
__device__ __forceinline__ void umma_pair_commit(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}

struct PairUnit {
  int mp, n_tile, g;
  int npass;
  int group[2];
  int mask[2];   // bit r set: CTA r stores its half in this pass
  int k_lo, k_hi;
};

__device__ __forceinline__ PairUnit decode_pair(const Args& a, int u, int num_m, int num_mp, int num_n) {
  PairUnit c;
  const int per_group = num_mp * num_n;
  c.g = 0;
  if (a.group_mode == 2) {
    c.g = u / per_group;
    u -= c.g * per_group;
  }
  const int pb = a.pair_band;
  const int band_tiles = pb * num_n;
  const int band = u / band_tiles;
  const int within = u - band * band_tiles;
  const int rows = min(pb, num_mp - band * pb);
  c.n_tile = within / rows;
  c.mp = band * pb + (within - c.n_tile * rows);
  c.k_lo = 0;
  c.k_hi = a.K;
  c.npass = 1;
  c.group[0] = c.group[1] = 0;
  c.mask[0] = 3;
  c.mask[1] = 0;
  if (a.group_mode == 1) {
    int g0 = a.tile_group[2 * c.mp];
    int g1 = (2 * c.mp + 1 < num_m) ? a.tile_group[2 * c.mp + 1] : -1;
    if (g0 < 0 || g0 >= a.num_groups) g0 = -1;
    if (g1 < 0 || g1 >= a.num_groups) g1 = -1;
    if (g0 == g1) {
      c.npass = g0 < 0 ? 0 : 1;
      c.group[0] = max(g0, 0);
    } else {
      c.npass = 0;
      if (g0 >= 0) {
        c.group[c.npass] = g0;
        c.mask[c.npass] = 1;
        ++c.npass;
      }
      if (g1 >= 0) {
        c.group[c.npass] = g1;
        c.mask[c.npass] = 2;
        ++c.npass;
      }
    }
  } else if (a.group_mode == 2) {
    c.group[0] = c.g;
    c.k_lo = a.k_begin[c.g];
    c.k_hi = min(a.k_end[c.g], a.K);
    if (c.k_hi < c.k_lo) c.k_hi = c.k_lo;
  }
  return c;
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
    mot_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const Args args) {
  extern __shared__ uint8_t smem_raw[];
  // the dynamic window starts at the same offset in both CTAs, so every object below has the same
  // shared-memory offset in the pair (the products and the remote barrier addresses rely on it)
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + P_STAGES * P_A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + P_STAGES * P_STAGE_BYTES);
  uint64_t* full_bar = bars;                      // [P_STAGES]  used in the even CTA
  uint64_t* empty_bar = bars + P_STAGES;          // [P_STAGES]  one per CTA
  uint64_t* acc_full = bars + 2 * P_STAGES;       // [2]         one per CTA
  uint64_t* acc_empty = bars + 2 * P_STAGES + 2;  // [2]         used in the even CTA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * P_STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();        // 0: issues the products
  const int pair = blockIdx.x >> 1;
  const int npairs = gridDim.x >> 1;

  int m_eff = args.M;
  if (args.m_rows_dev != nullptr) m_eff = min(m_eff, max(*args.m_rows_dev, 0));
  const int num_m = (m_eff + BM - 1) / BM;
  const int num_mp = (num_m + 1) / 2;
  const int num_n = (args.N + BN - 1) / BN;
  const int num_units = num_mp * num_n * (args.group_mode == 2 ? args.num_groups : 1);

  if (threadIdx.x == 0) {
    for (int i = 0; i < P_STAGES; ++i) {
      mbar_init(&full_bar[i], 1);
      mbar_init(&empty_bar[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 8);   // four epilogue warps of each CTA
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();     // both CTAs' barriers exist before anything of the peer touches them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int u = pair; u < num_units && ok; u += npairs) {
        const PairUnit pu = decode_pair(args, u, num_m, num_mp, num_n);
        const int m0 = pu.mp * (2 * BM) + (int)rank * BM;
        const int n0 = pu.n_tile * BN + (int)rank * P_BN_HALF;
        for (int ps = 0; ps < pu.npass && ok; ++ps) {
          const int grp = args.group_mode == 1 ? (ps == 0 ? pu.group[0] : pu.group[1]) : 0;
          for (int k0 = pu.k_lo; k0 < pu.k_hi; k0 += BK, ++it) {
            const int s = it % P_STAGES;
            const uint32_t ph = (it / P_STAGES) & 1;
            if (!mbar_wait_cl(&empty_bar[s], ph ^ 1, abort_flag, args.status, 1)) {
              ok = false;
              break;
            }
            if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * P_STAGE_BYTES);
            const uint32_t fb = mapa_shared(smem_u32(&full_bar[s]), 0);
            uint8_t* a_dst = sA + s * P_A_BYTES;
            uint8_t* b_dst = sB + s * P_B_BYTES;
            if (A_MN) {
#pragma unroll
              for (int i = 0; i < BM / 64; ++i)
                tma_pair_load_2d(a_dst + i * MN_CHUNK_BYTES, &tmA, fb, m0 + 64 * i, k0);
            } else {
              tma_pair_load_2d(a_dst, &tmA, fb, k0, m0);
            }
            if (B_MN) {
#pragma unroll
              for (int i = 0; i < P_BN_HALF / 64; ++i)
                tma_pair_load_3d(b_dst + i * MN_CHUNK_BYTES, &tmB, fb, n0 + 64 * i, k0, grp);
            } else {
              tma_pair_load_3d(b_dst, &tmB, fb, k0, n0, grp);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (even CTA only) ----------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
      uint32_t it = 0;
      uint32_t tile_it = 0;
      bool ok = true;
      for (int u = pair; u < num_units && ok; u += npairs) {
        const PairUnit pu = decode_pair(args, u, num_m, num_mp, num_n);
        for (int ps = 0; ps < pu.npass && ok; ++ps) {
          const int acc = tile_it & 1;
          const uint32_t acc_ph = (tile_it >> 1) & 1;
          if (!mbar_wait_cl(&acc_empty[acc], acc_ph ^ 1, abort_flag, args.status, 2)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + acc * BN;
          bool first = true;
          for (int k0 = pu.k_lo; k0 < pu.k_hi; k0 += BK, ++it) {
            const int s = it % P_STAGES;
            const uint32_t ph = (it / P_STAGES) & 1;
            if (!mbar_wait_cl(&full_bar[s], ph, abort_flag, args.status, 3)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint32_t a_addr = smem_u32(sA + s * P_A_BYTES);
            const uint32_t b_addr = smem_u32(sB + s * P_B_BYTES);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t da = A_MN ? make_smem_desc(a_addr + k * (UMMA_K * 128), MN_CHUNK_BYTES, 1024)
                                       : make_smem_desc(a_addr + k * (UMMA_K * 2), 0, 1024);
              const uint64_t db = B_MN ? make_smem_desc(b_addr + k * (UMMA_K * 128), MN_CHUNK_BYTES, 1024)
                                       : make_smem_desc(b_addr + k * (UMMA_K * 2), 0, 1024);
              umma_pair_bf16_ss(d_tmem, da, db, idesc, first ? 0u : 1u);
              first = false;
            }
            // the stage is reusable in both CTAs once these products retire
            umma_pair_commit(smem_u32(&empty_bar[s]));
            umma_pair_commit(mapa_shared(smem_u32(&empty_bar[s]), 1));
          }
          if (!ok) break;
          umma_pair_commit(smem_u32(&acc_full[acc]));
          umma_pair_commit(mapa_shared(smem_u32(&acc_full[acc]), 1));
          ++tile_it;
        }
      }
    }
  } else {
    // ------------------------------ epilogue (both CTAs) ----------------------------------
    const int quarter = warp & 3;
    uint32_t tile_it = 0;
    bool ok = true;
    for (int u = pair; u < num_units && ok; u += npairs) {
      const PairUnit pu = decode_pair(args, u, num_m, num_mp, num_n);
      for (int ps = 0; ps < pu.npass && ok; ++ps) {
        const int acc = tile_it & 1;
        const uint32_t acc_ph = (tile_it >> 1) & 1;
        if (!mbar_wait_cl(&acc_full[acc], acc_ph, abort_flag, args.status, 4)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const bool has_acc = pu.k_hi > pu.k_lo;
        const bool mine = ((ps == 0 ? pu.mask[0] : pu.mask[1]) >> rank) & 1;
        const int row = pu.mp * (2 * BM) + (int)rank * BM + quarter * 32 + lane;
        const bool row_ok = mine && row < args.M;
        const int n0 = pu.n_tile * BN;
        const long long c_off =
            (args.group_mode == 2 ? pu.g * args.c_group_stride : 0) + (long long)row * args.ldc;
        if (mine) {
#pragma unroll 1
        for (int ch = 0; ch < BN / 32; ++ch) {
          const int col0 = n0 + ch * 32;
          if (col0 >= args.N) break;  // warp-uniform
          uint32_t r[32];
          if (has_acc) {
            tmem_ld_32x32b_x32(tmem_base + acc * BN + ch * 32 + ((uint32_t)(quarter * 32) << 16), r);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0u;
          }
          __syncwarp();
          if (row_ok) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * args.alpha;
            const int ncols = min(32, args.N - col0);  // multiple of 8
            if (args.out_mode <= 1) {
              __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(args.C) + c_off + col0;
              const __nv_bfloat16* rp =
                  args.residual ? args.residual + (long long)row * args.ldr + col0 : nullptr;
#pragma unroll
              for (int j8 = 0; j8 < 4; ++j8) {
                if (j8 * 8 >= ncols) break;
                if (args.out_mode == 1) {
                  uint4 old = *reinterpret_cast<const uint4*>(cp + j8 * 8);
                  const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
                  for (int q = 0; q < 4; ++q) {
                    float2 f = __bfloat1622float2(o2[q]);
                    v[j8 * 8 + 2 * q] += f.x;
                    v[j8 * 8 + 2 * q + 1] += f.y;
                  }
                }
                if (rp) {
                  uint4 rr = *reinterpret_cast<const uint4*>(rp + j8 * 8);
                  const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rr);
#pragma unroll
                  for (int q = 0; q < 4; ++q) {
                    float2 f = __bfloat1622float2(r2[q]);
                    v[j8 * 8 + 2 * q] += f.x;
                    v[j8 * 8 + 2 * q + 1] += f.y;
                  }
                }
                uint4 o;
                o.x = pack_bf16x2(v[j8 * 8 + 0], v[j8 * 8 + 1]);
                o.y = pack_bf16x2(v[j8 * 8 + 2], v[j8 * 8 + 3]);
                o.z = pack_bf16x2(v[j8 * 8 + 4], v[j8 * 8 + 5]);
                o.w = pack_bf16x2(v[j8 * 8 + 6], v[j8 * 8 + 7]);
                *reinterpret_cast<uint4*>(cp + j8 * 8) = o;
              }
            } else {
              float* cp = reinterpret_cast<float*>(args.C) + c_off + col0;
#pragma unroll
              for (int j4 = 0; j4 < 8; ++j4) {
                if (j4 * 4 >= ncols) break;
                float4 o = make_float4(v[j4 * 4], v[j4 * 4 + 1], v[j4 * 4 + 2], v[j4 * 4 + 3]);
                if (args.out_mode == 3) {
                  float4 old = *reinterpret_cast<const float4*>(cp + j4 * 4);
                  o.x += old.x;
                  o.y += old.y;
                  o.z += old.z;
                  o.w += old.w;
                }
                *reinterpret_cast<float4*>(cp + j4 * 4) = o;
              }
            }
          }  // row_ok
          __syncwarp();
        }
        }  // mine
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_remote(mapa_shared(smem_u32(&acc_empty[acc]), 0));
        ++tile_it;
      }
    }
  }

  // ------------------------------ teardown ------------------------------------
  // Nobody leaves while the other CTA may still read this CTA's shared memory, arrive on its barriers
  // or write its tensor memory: every role above ends after a bounded time, then the pair meets here.
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && warp == 1) {
    uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) {
    }
  }
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace gemm

struct CommArgs {
  int gather_b = 0, num_copy_ctas = 0, world = 1, my_rank = 0;
  const long long* shard_ptrs = nullptr;
  void* staging = nullptr;
  int shard_rows = 0, chunk_rows = 0;
  int* gather_flags = nullptr;
  int gather_seq = 0;
  const long long* rs_ptrs = nullptr;
  int rs_rows = 0;
  const int* m_rows_dev = nullptr;   // rows of A / C in use (device scalar)
};

// 0: single-CTA kernel only; 1: the pair kernel where it applies (plain / grouped products without a fused
// collective).  Set with snu1_gemm_set_pair_mode.
static int g_pair_mode = 1;
static int g_pair_band = gemm::P_BAND;

template <bool A_MN, bool B_MN>
static int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const gemm::Args& args, long long units,
                       cudaStream_t stream) {
  using namespace gemm;
  static int max_pairs = -1;   // co-resident 2-CTA clusters of this instantiation
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = P_SMEM_BYTES;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (max_pairs < 0) {
    SNU1_CUDA_CHECK(cudaFuncSetAttribute(mot_gemm_pair_kernel<A_MN, B_MN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES));
    cfg.gridDim = dim3(2 * (num_sms() / 2), 1, 1);
    int n = 0;
    SNU1_CUDA_CHECK(cudaOccupancyMaxActiveClusters(&n, mot_gemm_pair_kernel<A_MN, B_MN>, &cfg));
    if (n < 1) {
      set_last_error("gemm: no 2-CTA cluster of the pair kernel fits on this device");
      return kHostBadArg;
    }
    max_pairs = n < num_sms() / 2 ? n : num_sms() / 2;
  }
  const int pairs = (int)(units < max_pairs ? units : max_pairs);
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  SNU1_CUDA_CHECK(cudaLaunchKernelEx(&cfg, mot_gemm_pair_kernel<A_MN, B_MN>, tmA, tmB, args));
  return kHostOk;
}

static int launch_gemm(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                       long long ldb, long long ldc, int a_mn, int b_mn, int group_mode,
                       int num_groups, const int* tile_group, const int* k_begin, const int* k_end,
                       long long b_group_stride, long long c_group_stride, int out_mode,
                       const void* residual, long long ldr, float alpha, long long a_rows,
                       long long b_rows, cudaStream_t stream, const CommArgs* comm = nullptr) {
  using namespace gemm;
  if (M <= 0 || N <= 0 || K < 0) {
    set_last_error("gemm: bad sizes M=%d N=%d K=%d", M, N, K);
    return kHostBadArg;
  }
  if ((N % 8) != 0 || (lda % 8) != 0 || (ldb % 8) != 0 || (ldc % (out_mode >= 2 ? 4 : 8)) != 0) {
    set_last_error("gemm: N, lda, ldb must be multiples of 8 and ldc of %d (N=%d lda=%lld ldb=%lld ldc=%lld)",
                   out_mode >= 2 ? 4 : 8, N, lda, ldb, ldc);
    return kHostBadArg;
  }
  if (!a_mn && (K % 8) != 0) {
    set_last_error("gemm: K must be a multiple of 8 for K-major operands (K=%d)", K);
    return kHostBadArg;
  }
  if (group_mode == 2 && !(a_mn && b_mn)) {
    set_last_error("gemm: group_mode 2 (weight gradient) needs MN-major operands");
    return kHostBadArg;
  }
  if (group_mode < 0 || group_mode > 2 || (group_mode != 0 && num_groups <= 0)) {
    set_last_error("gemm: bad group_mode %d / num_groups %d", group_mode, num_groups);
    return kHostBadArg;
  }
  if (residual != nullptr && out_mode != 0) {
    set_last_error("gemm: residual is only supported with out_mode 0");
    return kHostBadArg;
  }
  if (out_mode == 4 || out_mode == 5) {
    if (comm == nullptr || comm->rs_ptrs == nullptr || comm->rs_rows <= 0 || comm->world < 1 || comm->world > 8 ||
        (long long)comm->rs_rows * comm->world < M || group_mode != 0) {
      set_last_error("gemm: out_mode 4 / 5 need the owners' buffers and rows-per-rank covering M");
      return kHostBadArg;
    }
  } else if ((reinterpret_cast<uintptr_t>(C) & 15) != 0 ||
      (residual && (reinterpret_cast<uintptr_t>(residual) & 15) != 0)) {
    set_last_error("gemm: C and residual must be 16-byte aligned");
    return kHostBadArg;
  }
  const int G = group_mode == 0 ? 1 : num_groups;

  CUtensorMap tmA, tmB, tmBlocal;
  int rc;
  if (a_mn) {
    // A is [a_rows (reduction)][M], M contiguous
    uint64_t dims[2] = {(uint64_t)M, (uint64_t)a_rows};
    uint64_t strides[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {64, (uint32_t)BK};
    rc = encode_tmap_bf16(&tmA, A, 2, dims, strides, box);
  } else {
    // A is [a_rows (M)][K], K contiguous
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)a_rows};
    uint64_t strides[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {64, (uint32_t)BM};
    rc = encode_tmap_bf16(&tmA, A, 2, dims, strides, box);
  }
  if (rc != kHostOk) return rc;
  const bool fused_comm = comm != nullptr && (comm->gather_b || comm->rs_ptrs != nullptr);
  const bool use_pair = g_pair_mode != 0 && !fused_comm && out_mode <= 3;
  const int gB = group_mode == 1 ? G : 1;
  const uint64_t gstride_bytes = (uint64_t)(gB > 1 ? b_group_stride : (long long)b_rows * ldb) * 2;
  if (b_mn) {
    // B is [g][b_rows (reduction)][N], N contiguous
    uint64_t dims[3] = {(uint64_t)N, (uint64_t)b_rows, (uint64_t)gB};
    uint64_t strides[2] = {(uint64_t)ldb * 2, gstride_bytes};
    uint32_t box[3] = {64, (uint32_t)BK, 1};
    rc = encode_tmap_bf16(&tmB, B, 3, dims, strides, box);
  } else {
    // B is [g][b_rows (N)][K], K contiguous
    uint64_t dims[3] = {(uint64_t)K, (uint64_t)b_rows, (uint64_t)gB};
    uint64_t strides[2] = {(uint64_t)ldb * 2, gstride_bytes};
    uint32_t box[3] = {64, (uint32_t)(use_pair ? P_BN_HALF : BN), 1};
    rc = encode_tmap_bf16(&tmB, B, 3, dims, strides, box);
  }
  if (rc != kHostOk) return rc;
  tmBlocal = tmB;

  Args args;
  memset(&args, 0, sizeof(args));
  args.M = M;
  args.N = N;
  args.K = K;
  args.group_mode = group_mode;
  args.num_groups = G;
  args.tile_group = tile_group;
  args.k_begin = k_begin;
  args.k_end = k_end;
  args.C = C;
  args.ldc = ldc;
  args.c_group_stride = c_group_stride;
  args.out_mode = out_mode;
  args.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  args.ldr = ldr;
  args.alpha = alpha;
  args.status = device_status_word();
  args.pair_band = g_pair_band;

  const int num_m = (M + BM - 1) / BM;
  const int num_n = (N + BN - 1) / BN;
  const long long tiles = (long long)num_m * num_n * (group_mode == 2 ? G : 1);
  int grid = (int)(tiles < num_sms() ? tiles : num_sms());
  if (comm != nullptr) {
    args.world = comm->world;
    args.my_rank = comm->my_rank;
    args.m_rows_dev = comm->m_rows_dev;
    if (out_mode == 4 || out_mode == 5) {
      for (int r = 0; r < comm->world; ++r) args.rs_dst[r] = reinterpret_cast<float*>(comm->rs_ptrs[r]);
      args.rs_rows = comm->rs_rows;
    }
    if (comm->gather_b) {
      const int W = comm->world;
      if (a_mn || b_mn || group_mode != 0 || W < 1 || W > 8 || comm->shard_rows * W != N ||
          (N / W) % BN != 0 || comm->chunk_rows <= 0 || comm->shard_rows % comm->chunk_rows != 0 ||
          comm->num_copy_ctas < 1 || comm->num_copy_ctas >= num_sms() || (((long long)K * 2) % 16) != 0) {
        set_last_error("gemm: fused all-gather needs K-major operands, N = world * shard_rows with shard_rows a "
                       "multiple of 256 and of chunk_rows (N=%d world=%d shard_rows=%d chunk_rows=%d)",
                       N, W, comm->shard_rows, comm->chunk_rows);
        return kHostBadArg;
      }
      args.gather_b = 1;
      args.num_copy_ctas = comm->num_copy_ctas;
      for (int r = 0; r < W; ++r) args.shard[r] = reinterpret_cast<const void*>(comm->shard_ptrs[r]);
      args.staging = comm->staging;
      args.shard_rows = comm->shard_rows;
      args.chunk_rows = comm->chunk_rows;
      args.row_bytes = (long long)ldb * 2;
      args.gather_flags = comm->gather_flags;
      args.gather_seq = comm->gather_seq;
      const int gemm_ctas = num_sms() - comm->num_copy_ctas;
      grid = comm->num_copy_ctas + (int)(tiles < gemm_ctas ? tiles : gemm_ctas);
      uint64_t ldims[3] = {(uint64_t)K, (uint64_t)comm->shard_rows, 1};
      uint64_t lstr[2] = {(uint64_t)ldb * 2, (uint64_t)comm->shard_rows * ldb * 2};
      uint32_t lbox[3] = {64, (uint32_t)BN, 1};
      rc = encode_tmap_bf16(&tmBlocal, reinterpret_cast<const void*>(comm->shard_ptrs[comm->my_rank]), 3, ldims,
                            lstr, lbox);
      if (rc != kHostOk) return rc;
    }
  }

  if (use_pair) {
    const long long units = (long long)((num_m + 1) / 2) * num_n * (group_mode == 2 ? G : 1);
    if (!a_mn && !b_mn) rc = launch_pair<false, false>(tmA, tmB, args, units, stream);
    else if (!a_mn && b_mn) rc = launch_pair<false, true>(tmA, tmB, args, units, stream);
    else if (a_mn && !b_mn) rc = launch_pair<true, false>(tmA, tmB, args, units, stream);
    else rc = launch_pair<true, true>(tmA, tmB, args, units, stream);
    if (rc != kHostOk) return rc;
    SNU1_CUDA_CHECK(cudaGetLastError());
    return kHostOk;
  }

#define SNU1_LAUNCH_GEMM(AMN, BMN)                                                              \
  do {                                                                                          \
    SNU1_CUDA_CHECK(cudaFuncSetAttribute(mot_gemm_kernel<AMN, BMN>,                             \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,           \
                                         SMEM_BYTES));                                          \
    mot_gemm_kernel<AMN, BMN><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB, tmBlocal, args); \
  } while (0)

  if (!a_mn && !b_mn) SNU1_LAUNCH_GEMM(false, false);
  else if (!a_mn && b_mn) SNU1_LAUNCH_GEMM(false, true);
  else if (a_mn && !b_mn) SNU1_LAUNCH_GEMM(true, false);
  else SNU1_LAUNCH_GEMM(true, true);
#undef SNU1_LAUNCH_GEMM
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

}  // namespace snu1

// 1 (default): products without a fused collective run on the two-SM pair kernel (tcgen05 cta_group::2);
// 0: everything on the single-CTA kernel.  Returns the previous value.
SNU1_API int snu1_gemm_set_pair_mode(int mode) {
  const int old = snu1::g_pair_mode;
  snu1::g_pair_mode = mode != 0;
  return old;
}

// Pair tiles (256 rows each) per scheduling band of the pair kernel: all column tiles of one band are visited
// before the next band, so a band's rows of A stay in L2 while B streams once per band.  Returns the old value.
SNU1_API int snu1_gemm_set_pair_band(int band) {
  const int old = snu1::g_pair_band;
  if (band >= 1) snu1::g_pair_band = band;
  return old;
}

// C[M,N] (+)= alpha * op(A) op(B) (+ residual), bf16 inputs, fp32 accumulation.
//
//   a_mn = 0: A is [a_rows = M rows][K], row stride lda (K contiguous)
//   a_mn = 1: A is [a_rows = reduction rows][M], row stride lda (M contiguous)
//   b_mn = 0: B is [groups][b_rows = N rows][K], row stride ldb
//   b_mn = 1: B is [groups][b_rows = reduction rows][N], row stride ldb
//   group_mode 0: one problem.  1: tile_group[m_tile] selects the B group.
//   2: outputs C + g * c_group_stride reduce over rows [k_begin[g], k_end[g]).
//   out_mode 0 bf16 store (+ residual), 1 bf16 accumulate, 2 fp32 store, 3 fp32 accumulate.
SNU1_API int snu1_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K,
                            long long lda, long long ldb, long long ldc, int a_mn, int b_mn,
                            int group_mode, int num_groups, const int* tile_group,
                            const int* k_begin, const int* k_end, long long b_group_stride,
                            long long c_group_stride, int out_mode, const void* residual,
                            long long ldr, float alpha, long long a_rows, long long b_rows,
                            void* stream) {
  return snu1::launch_gemm(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, group_mode, num_groups,
                           tile_group, k_begin, k_end, b_group_stride, c_group_stride, out_mode,
                           residual, ldr, alpha, a_rows, b_rows,
                           reinterpret_cast<cudaStream_t>(stream));
}


// Same product for an A / C of M rows of which only *m_rows_dev (a device scalar) are in use: row tiles past
// that count are not visited.  For buffers sized for a worst case whose fill is only known on the device
// (expert-parallel receive buffers).  group_mode 0 / 1 only.
SNU1_API int snu1_gemm_bf16_rows(const void* A, const void* B, void* C, int M, int N, int K,
                                 long long lda, long long ldb, long long ldc, int a_mn, int b_mn,
                                 int group_mode, int num_groups, const int* tile_group, long long b_group_stride,
                                 int out_mode, float alpha, long long a_rows, long long b_rows,
                                 const int* m_rows_dev, void* stream) {
  if (group_mode == 2) {
    snu1::set_last_error("gemm_bf16_rows: the weight-gradient form has no row dimension to bound");
    return snu1::kHostBadArg;
  }
  snu1::CommArgs c;
  c.m_rows_dev = m_rows_dev;
  return snu1::launch_gemm(A, B, C, M, N, K, lda, ldb, ldc, a_mn, b_mn, group_mode, num_groups, tile_group, nullptr,
                           nullptr, b_group_stride, 0, out_mode, nullptr, 0, alpha, a_rows, b_rows,
                           reinterpret_cast<cudaStream_t>(stream), &c);
}

// y[M, N] = x[M,K] @ W^T where W [N,K] is split by rows over `world` GPUs: rank r holds rows
// [r * shard_rows, (r+1) * shard_rows) at shard_ptrs[r] (peer-mapped).  One kernel gathers the shards
// into `staging` [N,K] (local; this rank's own rows are read in place) and multiplies, shard by
// shard in ring order.  `flags` holds
// N / chunk_rows ints that must be < seq on entry; they equal seq on exit (reuse with seq + 1).
SNU1_API int snu1_gemm_allgather_bf16(const void* A, long long lda, int M, int K, const long long* shard_ptrs,
                                      int world, int my_rank, int shard_rows, void* staging, int* flags,
                                      int seq, int chunk_rows, int num_copy_ctas, void* C, long long ldc,
                                      int out_mode, const void* residual, long long ldr, void* stream) {
  snu1::CommArgs c;
  c.gather_b = 1;
  c.num_copy_ctas = num_copy_ctas;
  c.world = world;
  c.my_rank = my_rank;
  c.shard_ptrs = shard_ptrs;
  c.staging = staging;
  c.shard_rows = shard_rows;
  c.chunk_rows = chunk_rows;
  c.gather_flags = flags;
  c.gather_seq = seq;
  const int N = world * shard_rows;
  return snu1::launch_gemm(A, staging, C, M, N, K, lda, K, ldc, 0, 0, 0, 1, nullptr, nullptr, nullptr, 0, 0,
                           out_mode, residual, ldr, 1.0f, M, N, reinterpret_cast<cudaStream_t>(stream), &c);
}

// Reduce-scatter fused into the epilogue: the product's rows are owned by ranks in blocks of rs_rows; each
// tile is added with fp32 reductions into dst_ptrs[owner] ([rs_rows][ldc] fp32, must be zeroed and every rank
// must have finished before anyone reads).  Covers the weight-gradient reduce-scatter of weight parallelism
// (a_mn = b_mn = 1) and the row-parallel output reduce-scatter of tensor / sequence parallelism (a_mn = b_mn = 0).
SNU1_API int snu1_gemm_reducescatter_bf16(const void* A, const void* B, int M, int N, int K, long long lda,
                                          long long ldb, int a_mn, int b_mn, const long long* dst_ptrs, int world,
                                          int rs_rows, long long ldc, float alpha, long long a_rows,
                                          long long b_rows, void* stream) {
  snu1::CommArgs c;
  c.world = world;
  c.rs_ptrs = dst_ptrs;
  c.rs_rows = rs_rows;
  return snu1::launch_gemm(A, B, nullptr, M, N, K, lda, ldb, ldc, a_mn, b_mn, 0, 1, nullptr, nullptr, nullptr, 0,
                           0, 4, nullptr, 0, alpha, a_rows, b_rows, reinterpret_cast<cudaStream_t>(stream), &c);
}

// Staged form of the fused reduce-scatter: every rank stores its bf16 partial rows into slab `my_rank` of the
// owner's staging buffer (stage_ptrs[owner]: [world][rs_rows][ldc] bf16) from the GEMM epilogue.  After a
// barrier the owner calls snu1_sum_slabs to add its `world` slabs.  No atomics, half the wire bytes.
SNU1_API int snu1_gemm_reducescatter_staged_bf16(const void* A, const void* B, int M, int N, int K, long long lda,
                                                 long long ldb, int a_mn, int b_mn, const long long* stage_ptrs,
                                                 int world, int my_rank, int rs_rows, long long ldc, float alpha,
                                                 long long a_rows, long long b_rows, void* stream) {
  snu1::CommArgs c;
  c.world = world;
  c.my_rank = my_rank;
  c.rs_ptrs = stage_ptrs;
  c.rs_rows = rs_rows;
  return snu1::launch_gemm(A, B, nullptr, M, N, K, lda, ldb, ldc, a_mn, b_mn, 0, 1, nullptr, nullptr, nullptr, 0,
                           0, 5, nullptr, 0, alpha, a_rows, b_rows, reinterpret_cast<cudaStream_t>(stream), &c);
}

namespace snu1 {
// dst[i] (+)= sum over w of src[w * n + i]; src bf16, dst fp32 or bf16.
template <typename OT>
__global__ void __launch_bounds__(256)
    sum_slabs_kernel(const __nv_bfloat16* __restrict__ src, int world, long long n, OT* __restrict__ dst, int accumulate) {
  const long long nvec = n >> 3;
  for (long long iv = blockIdx.x * 256ll + threadIdx.x; iv < nvec; iv += (long long)gridDim.x * 256) {
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
    for (int w = 0; w < world; ++w) {
      const uint4 u = *reinterpret_cast<const uint4*>(src + (long long)w * n + (iv << 3));
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = __bfloat1622float2(h[e]);
        acc[2 * e] += f.x;
        acc[2 * e + 1] += f.y;
      }
    }
    if constexpr (sizeof(OT) == 4) {
      float4* d = reinterpret_cast<float4*>(dst + (iv << 3));
      float4 a = make_float4(acc[0], acc[1], acc[2], acc[3]), b = make_float4(acc[4], acc[5], acc[6], acc[7]);
      if (accumulate) {
        const float4 o0 = d[0], o1 = d[1];
        a.x += o0.x; a.y += o0.y; a.z += o0.z; a.w += o0.w;
        b.x += o1.x; b.y += o1.y; b.z += o1.z; b.w += o1.w;
      }
      d[0] = a;
      d[1] = b;
    } else {
      uint4* d = reinterpret_cast<uint4*>(dst + (iv << 3));
      if (accumulate) {
        const uint4 o = *d;
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&o);
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
      *d = o;
    }
  }
}
}  // namespace snu1

// out_dtype: 0 bf16, 1 fp32.  n must be a multiple of 8, pointers 16-byte aligned.
SNU1_API int snu1_sum_slabs(const void* src, int world, long long n, void* dst, int out_dtype, int accumulate,
                            void* stream) {
  if (n <= 0) return snu1::kHostOk;
  if ((n & 7) || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15) || world < 1) {
    snu1::set_last_error("sum_slabs: n must be a multiple of 8 and pointers 16-byte aligned");
    return snu1::kHostBadArg;
  }
  long long blocks = ((n >> 3) + 255) / 256;
  const int grid = (int)(blocks < 148 * 16 ? blocks : 148 * 16);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (out_dtype == 1)
    snu1::sum_slabs_kernel<float><<<grid, 256, 0, st>>>((const __nv_bfloat16*)src, world, n, (float*)dst, accumulate);
  else
    snu1::sum_slabs_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)src, world, n,
                                                                 (__nv_bfloat16*)dst, accumulate);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return snu1::kHostOk;
}
