// Data-movement kernels that do not fit the elementwise engine: batched 2-D transpose
// through shared-memory tiles and an inclusive prefix sum along the last dimension.
//
// The reference implements Permute / Transpose and Cumsum as host loops over index tuples
// (tensor/ops_shape.go, tensor/ops_extra.go).  Most permutes in this framework stay strided
// views (the GEMM and attention kernels take strides); these kernels serve the places that
// need a materialised transpose or a scan.
#include "common.cuh"

using namespace gb;

namespace {

// out[b][c][r] = in[b][r][c]; 32 x 32 tiles, 32 x 8 threads, padded shared tile.
template <typename T>
__global__ void transpose_kernel(const T* __restrict__ in, T* __restrict__ out, int R, int C) {
  __shared__ T tile[32][33];
  const long long b = blockIdx.z;
  const T* src = in + b * (long long)R * C;
  T* dst = out + b * (long long)R * C;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
#pragma unroll
  for (int k = 0; k < 32; k += 8) {
    const int r = r0 + threadIdx.y + k, c = c0 + threadIdx.x;
    if (r < R && c < C) tile[threadIdx.y + k][threadIdx.x] = src[(long long)r * C + c];
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 32; k += 8) {
    const int c = c0 + threadIdx.y + k, r = r0 + threadIdx.x;
    if (r < R && c < C) dst[(long long)c * R + r] = tile[threadIdx.x][threadIdx.y + k];
  }
}

template <typename T> struct ScanAcc { using CT = float; };
template <> struct ScanAcc<double> { using CT = double; };

// One CTA per row: the row is walked in chunks of blockDim.x * 4 elements; inside a chunk a
// thread scans its 4 elements, warps scan the thread totals by shuffles, a shared array
// carries the warp totals, and a running carry links the chunks.  Fixed order: deterministic.
template <typename T>
__global__ void __launch_bounds__(256)
cumsum_kernel(const T* __restrict__ x, T* __restrict__ y, long long n, int reverse) {
  using CT = typename ScanAcc<T>::CT;
  __shared__ CT warp_tot[8];
  __shared__ CT carry_s;
  const long long row = blockIdx.x;
  const T* xr = x + row * n;
  T* yr = y + row * n;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = CT(0);
  __syncthreads();
  for (long long base = 0; base < n; base += 1024) {
    CT v[4];
    CT run = CT(0);
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const long long i = base + threadIdx.x * 4 + j;
      const long long src = reverse ? n - 1 - i : i;
      v[j] = i < n ? (CT)xr[src] : CT(0);
      run += v[j];
      v[j] = run;
    }
    // inclusive scan of the thread totals inside the warp
    CT incl = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const CT up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    CT before = carry_s + (incl - run);
    for (int w = 0; w < warp; w++) before += warp_tot[w];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const long long i = base + threadIdx.x * 4 + j;
      if (i < n) yr[reverse ? n - 1 - i : i] = (T)(before + v[j]);
    }
    __syncthreads();
    if (threadIdx.x == 255) carry_s = before + run;
    __syncthreads();
  }
}

}  // namespace

enum { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2, DT_F64 = 3 };

// out[b][c][r] = in[b][r][c] for `batch` contiguous R x C matrices of `esize`-byte elements.
GB_EXPORT int gb_transpose2d(int esize, const void* in, void* out, int R, int C, int batch, void* stream) {
  if (R <= 0 || C <= 0 || batch <= 0) return gbh::E_OK;
  if (batch > 65535) {
    gbh::set_error("gb_transpose2d: at most 65535 matrices per call (got %d)", batch);
    return gbh::E_TOO_LARGE;
  }
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid((C + 31) / 32, (R + 31) / 32, batch), blk(32, 8);
  switch (esize) {
    case 2: transpose_kernel<unsigned short><<<grid, blk, 0, s>>>((const unsigned short*)in, (unsigned short*)out, R, C); break;
    case 4: transpose_kernel<unsigned int><<<grid, blk, 0, s>>>((const unsigned int*)in, (unsigned int*)out, R, C); break;
    case 8: transpose_kernel<unsigned long long><<<grid, blk, 0, s>>>((const unsigned long long*)in, (unsigned long long*)out, R, C); break;
    default:
      gbh::set_error("gb_transpose2d: element size %d is not supported", esize);
      return gbh::E_BAD_ARG;
  }
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

// Inclusive prefix sum along the last dimension of a (rows, n) tensor; reverse != 0 scans
// from the end (the adjoint of the forward scan).
GB_EXPORT int gb_cumsum(int dtype, const void* x, void* y, long long rows, long long n, int reverse, void* stream) {
  if (rows <= 0 || n <= 0) return gbh::E_OK;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case DT_BF16: cumsum_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n, reverse); break;
    case DT_F16: cumsum_kernel<__half><<<(unsigned)rows, 256, 0, s>>>((const __half*)x, (__half*)y, n, reverse); break;
    case DT_F32: cumsum_kernel<float><<<(unsigned)rows, 256, 0, s>>>((const float*)x, (float*)y, n, reverse); break;
    case DT_F64: cumsum_kernel<double><<<(unsigned)rows, 256, 0, s>>>((const double*)x, (double*)y, n, reverse); break;
    default:
      gbh::set_error("gb_cumsum: bad dtype %d", dtype);
      return gbh::E_BAD_ARG;
  }
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}
