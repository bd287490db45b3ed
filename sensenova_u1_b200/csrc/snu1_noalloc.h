// Allocation-free entry point of the native library.
//
// This entry point has no counterpart in the reference implementation: the
// reference is pure Python and leaves every device allocation to the PyTorch
// caching allocator.  It exists for callers of this library that are not allowed
// to allocate device memory at the point where they need the attention backward
// pass: code that runs inside a region where cudaMalloc is forbidden or would
// synchronise the whole device (a latency-critical serving loop, a plugin that
// only receives pre-allocated buffers from its host application, a process whose
// memory budget was handed out up front and whose allocator is locked afterwards).
//
// snu1_attn_bwd needs a scratch array delta[Hq][Sq] (fp32) that the caller must
// provide, and its status word is allocated lazily with cudaMalloc.  The variant
// below takes the same inputs and outputs, but keeps both the scratch and the
// status word in a fixed array inside the library image:
//
//   * capacity: Hq * Sq <= SNU1_NOALLOC_MAX_DELTA (1,048,576 floats, 4 MiB; for
//     example 32 heads x 32768 rows).  Larger problems are rejected with
//     SNU1_NOALLOC_TOO_LARGE (-4) and a message from snu1_last_error(); nothing is
//     launched in that case.
//   * the array is part of the library: every GPU that loads the library holds its
//     4 MiB + 256 B until the process exits, whether or not this function is called.
//   * no cudaMalloc / cudaFree / allocating library routine is called, neither on the
//     first call nor later.  The first call on each device looks the array's device
//     address up (cudaGetSymbolAddress) with that device current and remembers it;
//     make that first call outside of any stream capture.
//   * all calls share the one array and it keeps whatever the previous call left.  The
//     call itself rewrites every delta entry it reads and clears the status word first,
//     so back-to-back calls on ONE stream are fine; calls that can overlap on the GPU
//     (different streams, different host threads) race on it and must be serialised by
//     the caller.
//   * status_out (optional, host pointer, preferably pinned): receives the kernels'
//     status word (0 = ok) through a copy queued on `stream`; read it after the
//     stream has been synchronised.
#pragma once

#define SNU1_NOALLOC_MAX_DELTA (1 << 20)
#define SNU1_NOALLOC_TOO_LARGE (-4)

#ifdef __cplusplus
extern "C" {
#endif

int snu1_attn_bwd_noalloc(const void* q, long long ldq, const void* k, long long ldk, const void* v,
                          long long ldv, const void* o, long long ldo, const void* dout, long long lddo,
                          const float* lse, void* dq, long long lddq, void* dk, long long lddk, void* dv,
                          long long lddv, const void* meta_q, const void* meta_k, const int* kv_list,
                          const int* kv_count, const int* q_list, const int* q_count, int Sq, int Sk,
                          int Hq, int Hkv, float scale, int* status_out, void* stream);

#ifdef __cplusplus
}
#endif
