#include "host_common.h"

#include <stdarg.h>
#include <string.h>

#include <mutex>

namespace snu1 {

static thread_local char g_err[512] = {0};

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
const char* last_error() { return g_err; }

static constexpr int kMaxDevices = 64;
static int* g_status[kMaxDevices] = {nullptr};
static int g_sms[kMaxDevices] = {0};
static std::mutex g_mu;

int* device_status_word() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_status[dev] == nullptr) {
    int* p = nullptr;
    if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 256);
    g_status[dev] = p;
  }
  return g_status[dev];
}

int num_sms() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  if (g_sms[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    g_sms[dev] = n;
  }
  return g_sms[dev];
}

static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    }
  });
  return fn;
}

int encode_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                     const uint64_t* strides, const uint32_t* box) {
  auto fn = get_encode_fn();
  if (fn == nullptr) {
    set_last_error("cuTensorMapEncodeTiled is not available from this driver");
    return kHostTmap;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) {
    set_last_error("tensor map base %p is not 16-byte aligned", base);
    return kHostTmap;
  }
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bdim[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estr[i] = 1;
    if (i > 0) {
      gstr[i - 1] = strides[i - 1];
      if (strides[i - 1] % 16 != 0) {
        set_last_error("tensor map stride %llu is not a multiple of 16 bytes",
                       (unsigned long long)strides[i - 1]);
        return kHostTmap;
      }
    }
  }
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank),
                  const_cast<void*>(base), gdim, gstr, bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled failed with CUresult %d (rank %d dims %llu,%llu box %u,%u)",
                   (int)r, rank, (unsigned long long)dims[0], (unsigned long long)dims[1], box[0],
                   box[1]);
    return kHostTmap;
  }
  return kHostOk;
}

}  // namespace snu1

SNU1_API const char* snu1_last_error() { return snu1::last_error(); }

// Reads and clears the status word of the current device.  Synchronises the
// device.  Returns the status (0 = no kernel reported a problem).
SNU1_API int snu1_read_status(int* out_status) {
  int* p = snu1::device_status_word();
  if (p == nullptr) {
    snu1::set_last_error("no status word (cudaMalloc failed?)");
    return snu1::kHostCuda;
  }
  int v = 0;
  SNU1_CUDA_CHECK(cudaDeviceSynchronize());
  SNU1_CUDA_CHECK(cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost));
  if (v != 0) SNU1_CUDA_CHECK(cudaMemset(p, 0, sizeof(int)));
  *out_status = v;
  return snu1::kHostOk;
}

// Allocates the status word of the current device ahead of time so that no
// entry point allocates later (for instance under stream capture).
SNU1_API int snu1_init_device() {
  return snu1::device_status_word() != nullptr ? snu1::kHostOk : snu1::kHostCuda;
}
