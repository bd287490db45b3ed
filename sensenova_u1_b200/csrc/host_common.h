// Host-side helpers shared by the launchers: the per-device status word, TMA
// tensor-map encoding through the driver entry point (no link-time libcuda
// dependency), and error plumbing for the C ABI.
#pragma once
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define SNU1_API extern "C" __attribute__((visibility("default")))

namespace snu1 {

// Error codes returned by every extern "C" entry point.
enum HostError : int {
  kHostOk = 0,
  kHostBadArg = -1,
  kHostCuda = -2,
  kHostTmap = -3,
  kHostTooLarge = -4,
};

void set_last_error(const char* fmt, ...);
const char* last_error();

// Device status word of the current device (lazily cudaMalloc'ed, zeroed).
int* device_status_word();
int num_sms();

#define SNU1_CUDA_CHECK(expr)                                                          \
  do {                                                                                 \
    cudaError_t _e = (expr);                                                           \
    if (_e != cudaSuccess) {                                                           \
      ::snu1::set_last_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),   \
                             __FILE__, __LINE__);                                      \
      return ::snu1::kHostCuda;                                                        \
    }                                                                                  \
  } while (0)

// Encode a tiled bf16 tensor map with 128-byte swizzle.
//   rank      : 2..4
//   dims      : extents, innermost first (elements)
//   strides   : byte strides of dims[1..rank-1]
//   box       : box extents, innermost first (box[0] * 2 bytes must be 128)
// Returns kHostOk or kHostTmap.
int encode_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                     const uint64_t* strides, const uint32_t* box);

}  // namespace snu1
