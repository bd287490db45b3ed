// Index kernels of the convolutional pixel head ("ConvDecoder": pixel-shuffle 2 -> conv3x3 -> GELU -> pixel-shuffle 2
// -> conv3x3 -> pixel-shuffle r; reference training/sensenovavl/model/modules/fm_modules.py:44-61,
// src/sensenova_u1/models/neo_unify/modeling_fm_modules.py:573-591, run there by cuDNN through nn.Conv2d).
//
// Here each 3x3 convolution is ONE tcgen05 GEMM of this package (csrc/gemm_sm100.cu) on a patch matrix that the
// kernels below assemble, with the pixel shuffle folded into the gather so that no shuffled tensor is ever stored:
//
//   ps_im2col      x [h*w, 4C] (token-major rows, channels last)  ->  A [(2h)*(2w), 9*C]
//                  A[(Y,X), (dy*3+dx)*C + c] = x[(y', x'), 4c + 2i + j]  with  (Y+dy-1, X+dx-1) = (2y'+i, 2x'+j),
//                  zero outside the image (padding 1).  The convolution is then  out = A @ Wp^T  with the weight
//                  permuted once per step to [O, 3, 3, C].
//   ps_col2im      the adjoint: dx[(y,x), 4c+2i+j] = sum_{dy,dx} dA[(2y+i-dy+1, 2x+j-dx+1), (dy*3+dx)*C + c]
//                  (a gather too: no atomics, deterministic).
//   pixel_regroup  y [(4h)*(4w), 3*r*r] (second convolution's output, channels last)  <->  per-token pixel blocks
//                  [h*w, (4r)*(4r)*3] in (row, column, channel) order: the last pixel shuffle plus the token blocking
//                  of the flow-matching loss, forward and backward.
#include "host_common.h"
#include "sm100_common.cuh"

namespace snu1 {

__global__ void __launch_bounds__(256)
    ps_im2col_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ A, int h, int w, int C) {
  const int H2 = 2 * h, W2 = 2 * w;
  const long long total = (long long)H2 * W2 * 9 * C;
  for (long long idx = blockIdx.x * 256ll + threadIdx.x; idx < total; idx += (long long)gridDim.x * 256) {
    const int c = (int)(idx % C);
    long long r = idx / C;
    const int tap = (int)(r % 9);
    r /= 9;
    const int X = (int)(r % W2), Y = (int)(r / W2);
    const int yy = Y + tap / 3 - 1, xx = X + tap % 3 - 1;
    __nv_bfloat16 v = __float2bfloat16_rn(0.f);
    if (yy >= 0 && yy < H2 && xx >= 0 && xx < W2)
      v = x[((long long)(yy >> 1) * w + (xx >> 1)) * (4 * C) + 4 * c + 2 * (yy & 1) + (xx & 1)];
    A[idx] = v;
  }
}

__global__ void __launch_bounds__(256)
    ps_col2im_kernel(const __nv_bfloat16* __restrict__ dA, __nv_bfloat16* __restrict__ dx, int h, int w, int C,
                     int accumulate) {
  const int H2 = 2 * h, W2 = 2 * w;
  const long long total = (long long)h * w * 4 * C;
  for (long long idx = blockIdx.x * 256ll + threadIdx.x; idx < total; idx += (long long)gridDim.x * 256) {
    const int ch = (int)(idx % (4 * C));
    const long long tok = idx / (4 * C);
    const int xq = (int)(tok % w), yq = (int)(tok / w);
    const int c = ch >> 2, i = (ch >> 1) & 1, j = ch & 1;
    const int py = 2 * yq + i, px = 2 * xq + j;      // position in the shuffled image
    float acc = accumulate ? __bfloat162float(dx[idx]) : 0.f;
#pragma unroll
    for (int tap = 0; tap < 9; ++tap) {
      const int Y = py - (tap / 3) + 1, X = px - (tap % 3) + 1;     // output pixel that read this element with `tap`
      if (Y >= 0 && Y < H2 && X >= 0 && X < W2)
        acc += __bfloat162float(dA[((long long)Y * W2 + X) * (9 * C) + (long long)tap * C + c]);
    }
    dx[idx] = __float2bfloat16_rn(acc);
  }
}

// forward: tok[(ty,tx), ((sy*r+a)*(4r) + (sx*r+b))*3 + ch] = y[((4ty+sy)*(4w) + 4tx+sx), ch*r*r + a*r + b]
// backward (to_y != 0): the same index map read the other way.
__global__ void __launch_bounds__(256)
    pixel_regroup_kernel(__nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ tok, int h, int w, int r,
                         int to_y) {
  const int tp = 4 * r;
  const int D = tp * tp * 3;
  const long long total = (long long)h * w * D;
  for (long long idx = blockIdx.x * 256ll + threadIdx.x; idx < total; idx += (long long)gridDim.x * 256) {
    const int e = (int)(idx % D);
    const long long t = idx / D;
    const int tx = (int)(t % w), ty = (int)(t / w);
    const int ch = e % 3;
    const int q = (e / 3) % tp, p = (e / 3) / tp;            // pixel row / column inside the token
    const int sy = p / r, a = p % r, sx = q / r, b = q % r;
    const long long yi = ((long long)(4 * ty + sy) * (4 * w) + 4 * tx + sx) * (3 * r * r) + ch * r * r + a * r + b;
    if (to_y)
      y[yi] = tok[idx];
    else
      tok[idx] = y[yi];
  }
}

static int grid_for_total(long long total) {
  long long b = (total + 255) / 256;
  const long long cap = 148ll * 16;
  return (int)(b < 1 ? 1 : (b < cap ? b : cap));
}

}  // namespace snu1

using namespace snu1;

SNU1_API int snu1_ps_im2col(const void* x, void* A, int h, int w, int C, void* stream) {
  if (h <= 0 || w <= 0 || C <= 0) {
    set_last_error("ps_im2col: empty problem");
    return kHostBadArg;
  }
  ps_im2col_kernel<<<grid_for_total((long long)h * w * 36 * C), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (__nv_bfloat16*)A, h, w, C);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_ps_col2im(const void* dA, void* dx, int h, int w, int C, int accumulate, void* stream) {
  if (h <= 0 || w <= 0 || C <= 0) {
    set_last_error("ps_col2im: empty problem");
    return kHostBadArg;
  }
  ps_col2im_kernel<<<grid_for_total((long long)h * w * 4 * C), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dA, (__nv_bfloat16*)dx, h, w, C, accumulate);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}

SNU1_API int snu1_pixel_regroup(void* y, void* tok, int h, int w, int r, int to_y, void* stream) {
  if (h <= 0 || w <= 0 || r <= 0) {
    set_last_error("pixel_regroup: empty problem");
    return kHostBadArg;
  }
  pixel_regroup_kernel<<<grid_for_total((long long)h * w * 48 * r * r), 256, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)y, (__nv_bfloat16*)tok, h, w, r, to_y);
  SNU1_CUDA_CHECK(cudaGetLastError());
  return kHostOk;
}
