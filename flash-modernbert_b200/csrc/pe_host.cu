// Error recording, device probing and TMA descriptor construction for libpe_b200.so.
#include "pe_host.h"

#include <stdarg.h>
#include <string.h>

#include <mutex>

namespace pe {

static thread_local char g_last_error[512] = "";

void set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return PE_OK;
  set_last_error("%s failed: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
  return PE_ERR_CUDA;
}

int sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int set_max_dynamic_smem(const void* func, int bytes, bool max_carveout) {
  static std::mutex lock;
  static const void* done_func[256];
  static int done_dev[256];
  static int n_done = 0;
  int dev = 0;
  PE_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> guard(lock);
  for (int i = 0; i < n_done; ++i)
    if (done_func[i] == func && done_dev[i] == dev) return PE_OK;
  PE_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  if (max_carveout)
    PE_CUDA(cudaFuncSetAttribute(func, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 cudaSharedmemCarveoutMaxShared));
  if (n_done < 256) {  // beyond that the attribute is simply set again on every launch
    done_func[n_done] = func;
    done_dev[n_done] = dev;
    ++n_done;
  }
  return PE_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Bytes outside the tensor read as zero (FLOAT_OOB_FILL_NONE means "no NaN fill", i.e. zeros).
// The driver entry point is resolved through the runtime so that the library
// links against cudart only.
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tmap_bf16_2d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols,
                      uint64_t row_stride_elts, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) {
    set_last_error("cuTensorMapEncodeTiled could not be resolved from the driver");
    return PE_ERR_CUDA;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (row_stride_elts * 2) % 16 != 0 ||
      box_rows == 0 || box_rows > 256 || rows == 0 || cols == 0) {
    set_last_error("tensor map: base %p / row stride %llu elements / box rows %u not encodable",
                   base, (unsigned long long)row_stride_elts, box_rows);
    return PE_ERR_ARG;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_elts * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled returned %d (rows %llu cols %llu stride %llu box %u)",
                   (int)r, (unsigned long long)rows, (unsigned long long)cols,
                   (unsigned long long)row_stride_elts, box_rows);
    return PE_ERR_CUDA;
  }
  return PE_OK;
}

}  // namespace pe

extern "C" int pe_version(void) { return 100; }

extern "C" const char* pe_last_error(void) { return pe::g_last_error; }

extern "C" int pe_device_check(void) {
  int dev = 0;
  PE_CUDA(cudaGetDevice(&dev));
  int major = 0, minor = 0;
  PE_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  PE_CUDA(cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev));
  if (major != 10) {
    pe::set_last_error("device %d is sm_%d%d; this library carries sm_100a code only", dev, major,
                       minor);
    return PE_ERR_UNSUPPORTED;
  }
  if (pe::encode_fn() == nullptr) {
    pe::set_last_error("cuTensorMapEncodeTiled could not be resolved from the driver");
    return PE_ERR_CUDA;
  }
  return PE_OK;
}

extern "C" int pe_read_status(const int32_t* status, int32_t* code_out, void* stream) {
  PE_REQUIRE(status != nullptr, "pe_read_status: status is NULL");
  int32_t v = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  PE_CUDA(cudaMemcpyAsync(&v, status, sizeof(v), cudaMemcpyDeviceToHost, s));
  PE_CUDA(cudaStreamSynchronize(s));
  if (code_out != nullptr) *code_out = v;
  if (v != 0) {
    pe::set_last_error("device status word = %d", v);
    return PE_ERR_DEVICE;
  }
  return PE_OK;
}
