// Library runtime: status word, error text, tensor-map encoding, device facts.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace {

constexpr int kMaxDevices = 16;
int* g_status_dev[kMaxDevices] = {nullptr};
std::mutex g_mu;
thread_local char g_err[512] = "";

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

}  // namespace

namespace gbh {

const char* last_error() { return g_err; }

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int* status_ptr() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_status_dev[dev] == nullptr) {
    int* p = nullptr;
    if (cudaMalloc(&p, 4 * sizeof(int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 4 * sizeof(int));
    g_status_dev[dev] = p;
  }
  return g_status_dev[dev];
}

static int load_encode() {
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_encode) return E_OK;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || fn == nullptr || qres != cudaDriverEntryPointSuccess) {
    set_error("cuTensorMapEncodeTiled is not available from the driver");
    return E_NO_DRIVER;
  }
  g_encode = (EncodeTiledFn)fn;
  return E_OK;
}

int encode_tmap(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base,
                const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                CUtensorMapSwizzle swz) {
  int rc = load_encode();
  if (rc != E_OK) return rc;
  cuuint64_t gdim[5];
  cuuint64_t gstr[5];
  cuuint32_t bx[5];
  cuuint32_t es[5];
  for (int i = 0; i < rank; i++) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
  }
  for (int i = 0; i + 1 < rank; i++) gstr[i] = strides_bytes[i];
  if (((uintptr_t)base & 15) != 0) {
    set_error("tensor map base %p is not 16-byte aligned", base);
    return E_TMAP;
  }
  for (int i = 0; i + 1 < rank; i++) {
    if (gstr[i] % 16 != 0) {
      set_error("tensor map stride %d = %llu bytes is not a multiple of 16", i,
                (unsigned long long)gstr[i]);
      return E_TMAP;
    }
  }
  CUresult r = g_encode(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bx, es,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with code %d (rank %d, dims %llu,%llu,%llu box %u,%u,%u)",
              (int)r, rank, (unsigned long long)gdim[0], (unsigned long long)(rank > 1 ? gdim[1] : 0),
              (unsigned long long)(rank > 2 ? gdim[2] : 0), bx[0], rank > 1 ? bx[1] : 0,
              rank > 2 ? bx[2] : 0);
    return E_TMAP;
  }
  return E_OK;
}

}  // namespace gbh

GB_EXPORT const char* gb_last_error() { return gbh::last_error(); }

// Copies the 4-int status word of the current device to `out` (synchronises
// the device) and optionally clears it.
GB_EXPORT int gb_status_read(int* out, int clear) {
  int* p = gbh::status_ptr();
  if (!p) {
    gbh::set_error("no status word (no CUDA device?)");
    return gbh::E_CUDA;
  }
  GB_CUDA_OK(cudaDeviceSynchronize());
  GB_CUDA_OK(cudaMemcpy(out, p, 4 * sizeof(int), cudaMemcpyDeviceToHost));
  if (clear) GB_CUDA_OK(cudaMemset(p, 0, 4 * sizeof(int)));
  return gbh::E_OK;
}

// 1 when this library was compiled with -DGB_BOUNDS_CHECK (bounds.cuh), else 0.
GB_EXPORT int gb_bounds_checked_build() {
#ifdef GB_BOUNDS_CHECK
  return 1;
#else
  return 0;
#endif
}

GB_EXPORT int gb_sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  return n;
}

GB_EXPORT int gb_abi_version() { return 1; }

namespace {
struct Words10 { unsigned int u[2]; float f[8]; };
__global__ void set_words_kernel(unsigned int* up, float* fp, const Words10 w) {
  if (threadIdx.x < 2 && up) up[threadIdx.x] = w.u[threadIdx.x];
  if (threadIdx.x < 8 && fp) fp[threadIdx.x] = w.f[threadIdx.x];
}
}  // namespace

// Writes two 32-bit words to `words` and eight floats to `floats` (either may be null) in stream
// order.  The values travel as kernel arguments, so the caller's memory can be reused at once:
// this is how the per-step bases and optimizer scalars of a replayed CUDA graph are updated.
GB_EXPORT int gb_set_words(unsigned int* words, unsigned int w0, unsigned int w1, float* floats,
                           const float* f8, void* stream) {
  Words10 w;
  w.u[0] = w0; w.u[1] = w1;
  for (int i = 0; i < 8; i++) w.f[i] = f8 ? f8[i] : 0.f;
  set_words_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(words, f8 ? floats : nullptr, w);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}
