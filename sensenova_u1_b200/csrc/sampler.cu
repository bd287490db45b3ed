// Flow-matching sampler step, fused: velocity from the x-prediction of the
// conditional / unconditional (/ image-conditional) branches, classifier-free
// guidance with optional norm correction, Euler update of the latent pixels, and
// re-patchify of the new state into the 16x16 patch rows the pixel front-end reads
// at the next step.
//
// Reference (separate torch ops per step): src/sensenova_u1/models/neo_unify/
// modeling_neo_chat.py:1803-1851 (t2i), :1574-1677 (editing, three branches),
// optimized_scale :95-110, patchify / unpatchify :399-428.
//
// Layouts: x_pred [n_branch][T][D] bf16 (branch 0 conditional, 1 unconditional,
// 2 image-only conditional), z [T][D] fp32 with D = 3 * (m p)^2 in (row, col, channel)
// order, patches [T * m * m][3 * p * p] bf16 in (a, b | c, i, j) block-major order.
#include "host_common.h"
#include "sm100_common.cuh"

namespace snu1 {

enum CfgNorm : int { kNormNone = 0, kNormGlobal = 1, kNormChannel = 2, kNormZeroStar = 3 };

struct SamplerArgs {
  const __nv_bfloat16* x_pred;
  float* z;
  __nv_bfloat16* patches;
  float* stats;  // [4]: sum v_c^2, sum v_cfg^2, sum v_c.v_u, sum v_u^2 (whole sample); then [grid][4] partials
  int T, D, n_branch, patch, merge;
  float t, t_next, t_eps, cfg_scale, img_cfg_scale;
  int use_cfg, norm_mode, first_step;
};

__device__ __forceinline__ float block_sum_256(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) t += scratch[i];
  return t;
}

__device__ __forceinline__ void branch_velocities(const SamplerArgs& a, long long idx, float zi,
                                                  float inv_den, float& vc, float& vu, float& vi) {
  const long long plane = (long long)a.T * a.D;
  vc = (__bfloat162float(a.x_pred[idx]) - zi) * inv_den;
  vu = a.n_branch > 1 ? (__bfloat162float(a.x_pred[plane + idx]) - zi) * inv_den : vc;
  vi = a.n_branch > 2 ? (__bfloat162float(a.x_pred[2 * plane + idx]) - zi) * inv_den : vu;
}

__device__ __forceinline__ float plain_cfg(const SamplerArgs& a, float vc, float vu, float vi) {
  if (a.n_branch > 2) return vu + a.cfg_scale * (vc - vi) + a.img_cfg_scale * (vi - vu);
  return vu + a.cfg_scale * (vc - vu);
}

// pass 1 (only for the global / zero-star corrections): whole-sample sums
__global__ void __launch_bounds__(256) sampler_stats_kernel(const SamplerArgs a) {
  __shared__ float scratch[8];
  const float inv_den = 1.f / fmaxf(1.f - a.t, a.t_eps);
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int tok = blockIdx.x; tok < a.T; tok += gridDim.x) {
    for (int d = threadIdx.x; d < a.D; d += 256) {
      const long long idx = (long long)tok * a.D + d;
      float vc, vu, vi;
      branch_velocities(a, idx, a.z[idx], inv_den, vc, vu, vi);
      const float v = plain_cfg(a, vc, vu, vi);
      s0 += vc * vc;
      s1 += v * v;
      s2 += vc * vu;
      s3 += vu * vu;
    }
  }
  s0 = block_sum_256(s0, scratch);
  s1 = block_sum_256(s1, scratch);
  s2 = block_sum_256(s2, scratch);
  s3 = block_sum_256(s3, scratch);
  // per-block partials, summed in a fixed order by sampler_stats_finalize: the sums (and with them the
  // sampled image) are reproducible run to run and identical on every rank of a guidance-parallel group
  if (threadIdx.x == 0) {
    float* part = a.stats + 4 + 4 * blockIdx.x;
    part[0] = s0;
    part[1] = s1;
    part[2] = s2;
    part[3] = s3;
  }
}

__global__ void __launch_bounds__(256) sampler_stats_finalize(float* stats, int nblocks) {
  __shared__ float scratch[8];
  float s[4] = {0.f, 0.f, 0.f, 0.f};
  for (int b = threadIdx.x; b < nblocks; b += 256) {
#pragma unroll
    for (int j = 0; j < 4; ++j) s[j] += stats[4 + 4 * b + j];
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float t = block_sum_256(s[j], scratch);
    if (threadIdx.x == 0) stats[j] = t;
  }
}

// pass 2: one CTA per token
__global__ void __launch_bounds__(256) sampler_step_kernel(const SamplerArgs a) {
  __shared__ float scratch[8];
  const int tok = blockIdx.x;
  const float inv_den = 1.f / fmaxf(1.f - a.t, a.t_eps);
  const float dt = a.t_next - a.t;
  const int mp = a.merge * a.patch;
  float scale = 1.f, alpha = 1.f;
  if (a.use_cfg && a.norm_mode == kNormGlobal)
    scale = fminf(1.f, sqrtf(a.stats[0]) / (sqrtf(a.stats[1]) + 1e-8f));
  if (a.use_cfg && a.norm_mode == kNormZeroStar) alpha = a.stats[2] / (a.stats[3] + 1e-8f);
  if (a.use_cfg && a.norm_mode == kNormChannel) {
    float nc = 0.f, nv = 0.f;
    for (int d = threadIdx.x; d < a.D; d += 256) {
      const long long idx = (long long)tok * a.D + d;
      float vc, vu, vi;
      branch_velocities(a, idx, a.z[idx], inv_den, vc, vu, vi);
      const float v = plain_cfg(a, vc, vu, vi);
      nc += vc * vc;
      nv += v * v;
    }
    nc = block_sum_256(nc, scratch);
    nv = block_sum_256(nv, scratch);
    scale = fminf(1.f, sqrtf(nc) / (sqrtf(nv) + 1e-8f));
  }
  for (int d = threadIdx.x; d < a.D; d += 256) {
    const long long idx = (long long)tok * a.D + d;
    const float zi = a.z[idx];
    float vc, vu, vi;
    branch_velocities(a, idx, zi, inv_den, vc, vu, vi);
    float v;
    if (!a.use_cfg) {
      v = vc;
    } else if (a.norm_mode == kNormZeroStar) {
      v = a.first_step ? 0.f : (vu * alpha + a.cfg_scale * (vc - vu * alpha));
    } else {
      v = plain_cfg(a, vc, vu, vi) * scale;
    }
    const float zn = zi + dt * v;
    a.z[idx] = zn;
    if (a.patches) {
      // d = ((a*p + i) * mp + (b*p + j)) * 3 + c
      const int c = d % 3;
      const int col = (d / 3) % mp, rowp = d / (3 * mp);
      const int pa = rowp / a.patch, pi = rowp % a.patch;
      const int pb = col / a.patch, pj = col % a.patch;
      const long long prow = (long long)tok * a.merge * a.merge + pa * a.merge + pb;
      a.patches[prow * (3 * a.patch * a.patch) + (c * a.patch + pi) * a.patch + pj] = __float2bfloat16_rn(zn);
    }
  }
}

}  // namespace snu1

using namespace snu1;

// stats: kSamplerStatsFloats floats of scratch (4 sums + per-block partials), needed by the
// whole-sample corrections (global, cfg_zero_star).
SNU1_API int snu1_sampler_step(const void* x_pred, float* z, void* patches, float* stats, int T, int D,
                               int n_branch, int patch, int merge, float t, float t_next, float t_eps,
                               float cfg_scale, float img_cfg_scale, int use_cfg, int norm_mode,
                               int first_step, void* stream) {
  if (T <= 0 || D != 3 * patch * merge * patch * merge || n_branch < 1 || n_branch > 3) {
    set_last_error("sampler_step: bad sizes T=%d D=%d patch=%d merge=%d branches=%d", T, D, patch, merge,
                   n_branch);
    return kHostBadArg;
  }
  SamplerArgs a;
  a.x_pred = (const __nv_bfloat16*)x_pred;
  a.z = z;
  a.patches = (__nv_bfloat16*)patches;
  a.stats = stats;
  a.T = T;
  a.D = D;
  a.n_branch = n_branch;
  a.patch = patch;
  a.merge = merge;
  a.t = t;
  a.t_next = t_next;
  a.t_eps = t_eps;
  a.cfg_scale = cfg_scale;
  a.img_cfg_scale = img_cfg_scale;
  a.use_cfg = (use_cfg && n_branch > 1) ? 1 : 0;
  a.norm_mode = norm_mode;
  a.first_step = first_step;
  cudaStream_t st = (cudaStream_t)stream;
  if (a.use_cfg && (norm_mode == kNormGlobal || norm_mode == kNormZeroStar)) {
    if (stats == nullptr) {
      set_last_error("sampler_step: this cfg_norm needs the stats scratch");
      return kHostBadArg;
    }
    const int nb = T < 592 ? T : 592;
    sampler_stats_kernel<<<nb, 256, 0, st>>>(a);
    sampler_stats_finalize<<<1, 256, 0, st>>>(stats, nb);
  }
  sampler_step_kernel<<<T, 256, 0, st>>>(a);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}
