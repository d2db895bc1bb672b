// int8 quantisation support kernels: min / max reduction, affine q-parameters computed
// on the device (so dynamic quantisation needs no host round trip), quantise to int8
// with round-half-away-from-zero and clamping to [-128, 127], and fake quantisation
// with a clamped straight-through backward.
//
// Rules follow the reference (quant/quant.go:100-143): q = clamp(round(x / s) + zp);
// affine range nudged to include 0, scale = (max - min) / 255, zp = -128 - round(min / s)
// clamped, degenerate range -> (1, 0); symmetric scale = max|x| / 127.
#include "common.cuh"

using namespace gb;

namespace {

template <typename T>
__global__ void minmax_partial_kernel(const T* __restrict__ x, long long n, float* __restrict__ part) {
  __shared__ float red[32];
  float mn = INFINITY, mx = -INFINITY;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float v = (float)x[i];
    mn = fminf(mn, v);
    mx = fmaxf(mx, v);
  }
  mx = block_max(mx, red);
  mn = -block_max(-mn, red);
  if (threadIdx.x == 0) {
    part[2 * blockIdx.x] = mn;
    part[2 * blockIdx.x + 1] = mx;
  }
}

// out4: {min, max, scale, zero_point (as float)}; zp_int also written to zp_out
__global__ void qparams_kernel(const float* __restrict__ part, int nparts, int symmetric,
                               float* __restrict__ out4, int* __restrict__ zp_out) {
  __shared__ float red[32];
  float mn = INFINITY, mx = -INFINITY;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) {
    mn = fminf(mn, part[2 * i]);
    mx = fmaxf(mx, part[2 * i + 1]);
  }
  mx = block_max(mx, red);
  mn = -block_max(-mn, red);
  if (threadIdx.x == 0) {
    float scale;
    int zp = 0;
    if (symmetric) {
      float m = fmaxf(fabsf(mn), fabsf(mx));
      scale = m == 0.f ? 1.f : m / 127.f;
    } else {
      float lo = fminf(0.f, mn), hi = fmaxf(0.f, mx);
      scale = (hi - lo) / 255.f;
      if (scale == 0.f) {
        scale = 1.f;
        zp = 0;
      } else {
        zp = -128 - (int)roundf(lo / scale);
        zp = zp < -128 ? -128 : (zp > 127 ? 127 : zp);
      }
    }
    out4[0] = mn; out4[1] = mx; out4[2] = scale; out4[3] = (float)zp;
    if (zp_out) *zp_out = zp;
  }
}

template <typename T>
__global__ void quantize_kernel(const T* __restrict__ x, int8_t* __restrict__ q, long long rows,
                                long long cols, long long ldq, const float* __restrict__ scale,
                                const int* __restrict__ zp, int per_row) {
  const long long n = rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols, c = i - r * cols;
    const float s = per_row ? scale[r] : scale[0];
    const int z = zp ? (per_row ? zp[r] : zp[0]) : 0;
    int v = (int)roundf((float)x[i] / s) + z;
    v = v < -128 ? -128 : (v > 127 ? 127 : v);
    q[r * ldq + c] = (int8_t)v;
  }
}

// Sixteen elements per thread: 16-byte stores of the int8 output, 16-byte loads of the input.
// Needs cols and ldq to be multiples of 16 and both base pointers 16-byte aligned, so that a
// group of sixteen never straddles a row.
template <typename T>
__global__ void quantize_vec_kernel(const T* __restrict__ x, int8_t* __restrict__ q, long long rows,
                                    long long cols, long long ldq, const float* __restrict__ scale,
                                    const int* __restrict__ zp, int per_row) {
  const long long groups = rows * cols / 16;
  const long long gpr = cols / 16;
  constexpr int LD = 16 / (int)sizeof(T);          // elements per 16-byte load
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < groups;
       g += (long long)gridDim.x * blockDim.x) {
    const long long r = g / gpr, c = (g - r * gpr) * 16;
    const float s = per_row ? scale[r] : scale[0];
    const int z = zp ? (per_row ? zp[r] : zp[0]) : 0;
    alignas(16) T v[16];
#pragma unroll
    for (int k = 0; k < 16 / LD; ++k)
      *reinterpret_cast<uint4*>(&v[k * LD]) = *reinterpret_cast<const uint4*>(x + r * cols + c + k * LD);
    alignas(16) int8_t o[16];
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      int w = (int)roundf((float)v[k] / s) + z;
      o[k] = (int8_t)(w < -128 ? -128 : (w > 127 ? 127 : w));
    }
    *reinterpret_cast<uint4*>(q + r * ldq + c) = *reinterpret_cast<const uint4*>(o);
  }
}

// MODE 0: y = (q(x) - zp) * s;  MODE 1: dx = dy where x lies inside the representable range
template <typename T, int MODE>
__global__ void fake_quant_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ y,
                                  long long n, const float* __restrict__ qp) {
  const float s = qp[0];
  const int zp = (int)qp[1];
  const float lo = (-128.f - zp) * s, hi = (127.f - zp) * s;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = (float)x[i];
    if (MODE == 0) {
      int q = (int)roundf(v / s) + zp;
      q = q < -128 ? -128 : (q > 127 ? 127 : q);
      y[i] = (T)((float)(q - zp) * s);
    } else {
      y[i] = (v >= lo && v <= hi) ? dy[i] : (T)0.f;
    }
  }
}

inline int grid_for(long long n) {
  long long g = (n + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  return g < 1 ? 1 : (int)g;
}

}  // namespace

enum { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2 };

#define GB_Q_DISPATCH(CALL)                                   \
  switch (dtype) {                                            \
    case DT_BF16: { using T = __nv_bfloat16; CALL; } break;   \
    case DT_F16: { using T = __half; CALL; } break;           \
    case DT_F32: { using T = float; CALL; } break;            \
    default:                                                  \
      gbh::set_error("quant: unsupported dtype %d", dtype);   \
      return gbh::E_BAD_ARG;                                  \
  }

GB_EXPORT int gb_q_scratch_floats() { return 2 * 148 * 8; }

// Observes x: out4 = {min, max, scale, zero_point}; zp_out (int, may be null) gets the
// zero point.  scratch: gb_q_scratch_floats() floats.
GB_EXPORT int gb_q_observe(int dtype, const void* x, long long n, int symmetric, float* scratch,
                           float* out4, int* zp_out, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  const int g = grid_for(n);
  GB_Q_DISPATCH((minmax_partial_kernel<T><<<g, 256, 0, s>>>((const T*)x, n, scratch)));
  qparams_kernel<<<1, 256, 0, s>>>(scratch, g, symmetric, out4, zp_out);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

// q[r][c] = clamp(round(x[r][c] / scale) + zp); scale / zp are device scalars, or one
// value per row when per_row != 0; zp may be null (0).  ldq: row pitch of q in bytes.
GB_EXPORT int gb_q_quantize(int dtype, const void* x, void* q, long long rows, long long cols,
                            long long ldq, const float* scale, const int* zp, int per_row,
                            void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (rows * cols <= 0) return gbh::E_OK;
  const bool vec = cols % 16 == 0 && ldq % 16 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)q & 15) == 0;
  if (vec) {
    GB_Q_DISPATCH((quantize_vec_kernel<T><<<grid_for(rows * cols / 16), 256, 0, s>>>((const T*)x, (int8_t*)q, rows, cols, ldq, scale, zp, per_row)));
  } else {
    GB_Q_DISPATCH((quantize_kernel<T><<<grid_for(rows * cols), 256, 0, s>>>((const T*)x, (int8_t*)q, rows, cols, ldq, scale, zp, per_row)));
  }
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

// mode 0: fake-quantise x into y; mode 1: straight-through gradient (x, dy -> y).
// qp: device pair {scale, zero_point as float}.
GB_EXPORT int gb_fake_quant(int mode, int dtype, const void* x, const void* dy, void* y, long long n,
                            const float* qp, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (n <= 0) return gbh::E_OK;
  if (mode == 0) {
    GB_Q_DISPATCH((fake_quant_kernel<T, 0><<<grid_for(n), 256, 0, s>>>((const T*)x, nullptr, (T*)y, n, qp)));
  } else {
    GB_Q_DISPATCH((fake_quant_kernel<T, 1><<<grid_for(n), 256, 0, s>>>((const T*)x, (const T*)dy, (T*)y, n, qp)));
  }
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}
