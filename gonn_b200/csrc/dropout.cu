// Inverted dropout with Philox-4x32-10: element i keeps its value (scaled by
// 1/(1-p)) when the random word derived from (seed, offset, i / 4) lane i % 4 is
// >= p * 2^32.  Forward and backward call the same kernel with the same
// (seed, offset), so no mask is stored.  The reference draws a host mask from
// the global RNG (nn/dropout.go:21-37).
#include "common.cuh"

using namespace gb;

namespace {

__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; r++) {
    uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}

template <typename T>
__global__ void dropout_kernel(const T* __restrict__ x, T* __restrict__ y, long long n, float p,
                               unsigned long long seed, unsigned long long offset) {
  const uint32_t thresh = (uint32_t)fminf(p * 4294967296.f, 4294967295.f);
  const float scale = 1.f / (1.f - p);
  const long long groups = (n + 3) / 4;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < groups;
       g += (long long)gridDim.x * blockDim.x) {
    uint4 r = philox4x32_10(make_uint4((uint32_t)g, (uint32_t)(g >> 32), (uint32_t)offset, (uint32_t)(offset >> 32)),
                            make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
    const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const long long i = g * 4 + j;
      if (i < n) y[i] = rr[j] >= thresh ? (T)((float)x[i] * scale) : (T)0.f;
    }
  }
}

// The same mask (element i still takes lane i % 4 of the draw for group i / 4) with 16-byte loads and
// stores: a thread handles 16 / sizeof(T) consecutive elements, i.e. one draw for fp32 and two for the
// 16-bit types.  Needs n to be a multiple of that count and 16-byte aligned pointers.
template <typename T>
__global__ void dropout_vec_kernel(const T* __restrict__ x, T* __restrict__ y, long long nvec, float p,
                                   unsigned long long seed, unsigned long long offset) {
  constexpr int V = 16 / (int)sizeof(T);      // 4 or 8
  const uint32_t thresh = (uint32_t)fminf(p * 4294967296.f, 4294967295.f);
  const float scale = 1.f / (1.f - p);
  const uint2 key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  uint4* yv = reinterpret_cast<uint4*>(y);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    uint4 u = xv[i];
    T* e = reinterpret_cast<T*>(&u);
#pragma unroll
    for (int h = 0; h < V / 4; h++) {
      const long long g = i * (V / 4) + h;
      const uint4 r = philox4x32_10(make_uint4((uint32_t)g, (uint32_t)(g >> 32), (uint32_t)offset, (uint32_t)(offset >> 32)), key);
      const uint32_t rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int j = 0; j < 4; j++) e[4 * h + j] = rr[j] >= thresh ? (T)((float)e[4 * h + j] * scale) : (T)0.f;
    }
    yv[i] = u;
  }
}

}  // namespace

enum { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2 };

GB_EXPORT int gb_dropout(int dtype, const void* x, void* y, long long n, float p, long long seed,
                         long long offset, void* stream) {
  if (n <= 0) return gbh::E_OK;
  long long g = ((n + 3) / 4 + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  cudaStream_t s = (cudaStream_t)stream;
  const int V = dtype == DT_F32 ? 4 : 8;
  if ((n % V) == 0 && ((((uintptr_t)x | (uintptr_t)y) & 15) == 0) && dtype >= DT_BF16 && dtype <= DT_F32) {
    const long long nvec = n / V;
    long long gv = (nvec + 255) / 256;
    if (gv > 148 * 16) gv = 148 * 16;
    if (dtype == DT_BF16) dropout_vec_kernel<__nv_bfloat16><<<(int)gv, 256, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, nvec, p, seed, offset);
    else if (dtype == DT_F16) dropout_vec_kernel<__half><<<(int)gv, 256, 0, s>>>((const __half*)x, (__half*)y, nvec, p, seed, offset);
    else dropout_vec_kernel<float><<<(int)gv, 256, 0, s>>>((const float*)x, (float*)y, nvec, p, seed, offset);
    GB_CUDA_OK(cudaGetLastError());
    return gbh::E_OK;
  }
  switch (dtype) {
    case DT_BF16: dropout_kernel<__nv_bfloat16><<<(int)g, 256, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n, p, seed, offset); break;
    case DT_F16: dropout_kernel<__half><<<(int)g, 256, 0, s>>>((const __half*)x, (__half*)y, n, p, seed, offset); break;
    case DT_F32: dropout_kernel<float><<<(int)g, 256, 0, s>>>((const float*)x, (float*)y, n, p, seed, offset); break;
    default:
      gbh::set_error("gb_dropout: bad dtype %d", dtype);
      return gbh::E_BAD_ARG;
  }
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}
