// Online-softmax merge of attention partial results: the step that lets attention over a key/value
// set split into blocks (one block per context-parallel rank) be computed block by block.
//
//   lse' = log2(2^lse_a + 2^lse_b),   o' = o_a 2^(lse_a - lse') + o_b 2^(lse_b - lse')
//
// lse is in log2 units ([heads][S] fp32, +inf = "this row saw no key", the convention of the
// attention forward kernel); the running output is kept in fp32 so that merging W blocks rounds
// once.  Reference: _update_out_and_lse (sigmoid / logsigmoid form on natural-log lse),
// training/sensenovalm/model/ops/ring_flash_attn/utils.py:20-58.
#include "host_common.h"
#include "sm100_common.cuh"

namespace snu1 {

// one warp per (row, head); 128 channels = 4 per lane
__global__ void __launch_bounds__(256)
    ring_merge_kernel(float* __restrict__ o_acc, float* __restrict__ lse_acc, const __nv_bfloat16* __restrict__ o_blk,
                      long long ld_blk, const float* __restrict__ lse_blk, __nv_bfloat16* __restrict__ out,
                      long long ld_out, int S, int H, int first) {
  const long long w = (blockIdx.x * 256ll + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long long)S * H) return;
  const int row = (int)(w / H), head = (int)(w - (long long)row * H);
  const float inf = __int_as_float(0x7f800000);
  const float lb = lse_blk[(long long)head * S + row];
  const float la = first ? inf : lse_acc[(long long)head * S + row];
  const bool has_a = la != inf, has_b = lb != inf;
  float wa = 0.f, wb = 0.f, ln = inf;
  if (has_a && has_b) {
    const float mx = fmaxf(la, lb);
    const float ea = exp2f(la - mx), eb = exp2f(lb - mx);
    ln = mx + log2f(ea + eb);
    wa = ea / (ea + eb);
    wb = eb / (ea + eb);
  } else if (has_a) {
    wa = 1.f;
    ln = la;
  } else if (has_b) {
    wb = 1.f;
    ln = lb;
  }
  float4* acc = reinterpret_cast<float4*>(o_acc + ((long long)row * H + head) * 128) + lane;
  const uint2 u = *(reinterpret_cast<const uint2*>(o_blk + (long long)row * ld_blk + head * 128) + lane);
  const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&u);
  const float2 b0 = __bfloat1622float2(hb[0]), b1 = __bfloat1622float2(hb[1]);
  float4 a = first ? make_float4(0.f, 0.f, 0.f, 0.f) : *acc;
  a.x = a.x * wa + b0.x * wb;
  a.y = a.y * wa + b0.y * wb;
  a.z = a.z * wa + b1.x * wb;
  a.w = a.w * wa + b1.y * wb;
  *acc = a;
  if (lane == 0) lse_acc[(long long)head * S + row] = ln;
  if (out != nullptr) {
    uint2 o;
    o.x = pack_bf16x2(a.x, a.y);
    o.y = pack_bf16x2(a.z, a.w);
    *(reinterpret_cast<uint2*>(out + (long long)row * ld_out + head * 128) + lane) = o;
  }
}

}  // namespace snu1

using namespace snu1;

// o_acc [S][H][128] fp32 and lse_acc [H][S] fp32 are the running result (ignored on input when first != 0);
// o_blk / lse_blk the block to merge in; out (optional) receives the merged output in bf16.
SNU1_API int snu1_ring_merge(float* o_acc, float* lse_acc, const void* o_blk, long long ld_blk, const float* lse_blk,
                             void* out, long long ld_out, int S, int H, int first, void* stream) {
  if (S <= 0 || H <= 0 || (ld_blk & 3) || (ld_out & 3)) {
    set_last_error("ring_merge: bad sizes S=%d H=%d ld=%lld/%lld", S, H, ld_blk, ld_out);
    return kHostBadArg;
  }
  const long long warps = (long long)S * H;
  ring_merge_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      o_acc, lse_acc, (const __nv_bfloat16*)o_blk, ld_blk, lse_blk, (__nv_bfloat16*)out, ld_out, S, H, first);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}
