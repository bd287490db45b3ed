// Shared pieces of the packed mixed-mask attention kernels.
//
// Mask model (training: training/sensenovavl/model/sensenovavl_moe_chat/
// modeling_sensenovavl_chat_mot.py:140-212; inference prefix:
// src/sensenova_u1/models/neo_unify/modeling_qwen3.py:157-180).  Every token
// carries (doc, pos, img, flags); flags bit0 = generation-branch token, bit1 =
// "never attend to this key".  A query q may attend to key k when
//
//   doc[q] == doc[k]
//   and (pos[q] >= pos[k]  or  (img[q] > 0 and img[q] == img[k]))
//   and (not gen[k]  or  (gen[q] and img[q] == img[k]))
//   and (not gen[q]  or  gen[k]  or  pos[k] != pos[q])
//   and not blocked[k]
//
// "Causal" is by pos, not by storage order (all tokens of an image share one
// pos, so an image is bidirectional), which is why the kernels work from a
// per-(query tile, key tile) classification {skip, partial, full} instead of a
// diagonal.
#pragma once
#include "sm100_common.cuh"

namespace snu1 {

struct TokMeta {  // 16 bytes, loaded as int4
  int doc;
  int pos;
  int img;
  int flags;
};

constexpr int kFlagGen = 1;
constexpr int kFlagBlocked = 2;

__device__ __forceinline__ bool mask_allowed(const TokMeta& q, const TokMeta& k) {
  const bool same_doc = q.doc == k.doc;
  const bool same_img = q.img > 0 && q.img == k.img;
  const bool base = same_doc && (q.pos >= k.pos || same_img);
  const bool gen_q = (q.flags & kFlagGen) != 0;
  const bool gen_k = (k.flags & kFlagGen) != 0;
  const bool gate1 = !gen_k || (gen_q && q.img == k.img);
  const bool gate2 = !gen_q || gen_k || k.pos != q.pos;
  return base && gate1 && gate2 && (k.flags & kFlagBlocked) == 0;
}

// Mask words of one row against 32 * NW consecutive columns, by the rule (fallback when a pair has no slot).
// ``row_is_query``: the row is a query and the columns are keys; otherwise the row is a key and the columns
// are queries.  Columns at or beyond ``cmax`` get zero bits.
template <int NW>
__device__ __forceinline__ void mask_words_by_rule(const TokMeta& row, const TokMeta* __restrict__ cols, int cmax,
                                                   bool row_is_query, uint32_t (&w)[NW]) {
  const int4* mc = reinterpret_cast<const int4*>(cols);
#pragma unroll
  for (int g = 0; g < NW; ++g) {
    uint32_t ww = 0u;
#pragma unroll 8
    for (int c = 0; c < 32; ++c) {
      const int i = g * 32 + c;
      bool allow = false;
      if (i < cmax) {
        const int4 t = __ldg(mc + i);
        const TokMeta o{t.x, t.y, t.z, t.w};
        allow = row_is_query ? mask_allowed(row, o) : mask_allowed(o, row);
      }
      ww |= (allow ? 1u : 0u) << c;
    }
    w[g] = ww;
  }
}

constexpr int kTileSkip = 0;
constexpr int kTilePartial = 1;
constexpr int kTileFull = 2;

// Tile lists: entry = tile index | (class << 24)
__device__ __forceinline__ int list_tile(int e) { return e & 0xffffff; }
__device__ __forceinline__ int list_class(int e) { return e >> 24; }

// named barrier among a subset of the CTA's threads
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 3-input maximum and packed two-lane fp32 arithmetic (sm_100): half the issue slots of the scalar forms
// in the softmax inner loops.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}

__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

}  // namespace snu1
