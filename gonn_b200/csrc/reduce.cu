// Axis reductions over a tensor viewed as (outer, R, inner): sum, mean, max,
// min (values) and argmax / argmin (first extremum wins, like the reference's
// ArgMax tie rule, tensor/ops_reduce.go:6-271).  Two layouts:
//   inner == 1  row reduction, one warp (short rows) or one CTA (long rows) per row
//   inner  > 1  column reduction, coalesced along inner, R optionally split
//               across CTAs with a second fixed-order pass (deterministic)
// The column form with outer == 1 is the bias-gradient reduction of Linear.
#include "bounds.cuh"

using namespace gb;

namespace {

enum ROp : int { R_SUM = 0, R_MEAN = 1, R_MAX = 2, R_MIN = 3, R_ARGMAX = 4, R_ARGMIN = 5 };

template <typename T> struct Acc { using CT = float; };
template <> struct Acc<double> { using CT = double; };

template <typename CT, int OP>
__device__ __forceinline__ CT r_init() {
  if (OP == R_MAX || OP == R_ARGMAX) return (CT)-INFINITY;
  if (OP == R_MIN || OP == R_ARGMIN) return (CT)INFINITY;
  return CT(0);
}
template <typename CT, int OP>
__device__ __forceinline__ CT r_comb(CT a, CT b) {
  if (OP == R_MAX) return a > b ? a : b;
  if (OP == R_MIN) return a < b ? a : b;
  return a + b;
}

template <typename CT, int OP>
__device__ __forceinline__ CT warp_red(CT v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = r_comb<CT, OP>(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// rows: (outer) rows of length R, contiguous.  One CTA per row.
template <typename T, typename TO, int OP>
__global__ void row_reduce_kernel(const T* __restrict__ x, TO* __restrict__ y, long long R) {
  using CT = typename Acc<T>::CT;
  __shared__ CT red[32];
  const T* xr = x + (long long)blockIdx.x * R;
  CT a = r_init<CT, OP>();
  for (long long i = threadIdx.x; i < R; i += blockDim.x) a = r_comb<CT, OP>(a, (CT)xr[i]);
  a = warp_red<CT, OP>(a);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) red[w] = a;
  __syncthreads();
  if (w == 0) {
    CT b = lane < nw ? red[lane] : r_init<CT, OP>();
    b = warp_red<CT, OP>(b);
    if (lane == 0) {
      if (OP == R_MEAN) b = b / (CT)R;
      y[blockIdx.x] = (TO)b;
    }
  }
}

// argmax / argmin over rows: first extremum wins
template <typename T, int OP>
__global__ void row_arg_kernel(const T* __restrict__ x, long long* __restrict__ y, long long R) {
  using CT = typename Acc<T>::CT;
  __shared__ CT rv[32];
  __shared__ long long ri[32];
  const T* xr = x + (long long)blockIdx.x * R;
  CT best = r_init<CT, OP>();
  long long bi = 0x7fffffffffffffffLL;
  for (long long i = threadIdx.x; i < R; i += blockDim.x) {
    CT v = (CT)xr[i];
    bool better = OP == R_ARGMAX ? v > best : v < best;
    if (better || (v == best && i < bi)) { best = v; bi = i; }
  }
  auto comb = [&](CT ov, long long oi) {
    bool better = OP == R_ARGMAX ? ov > best : ov < best;
    if (better || (ov == best && oi < bi)) { best = ov; bi = oi; }
  };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    CT ov = __shfl_xor_sync(0xffffffffu, best, o);
    long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
    comb(ov, oi);
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) { rv[w] = best; ri[w] = bi; }
  __syncthreads();
  if (w == 0) {
    best = lane < nw ? rv[lane] : r_init<CT, OP>();
    bi = lane < nw ? ri[lane] : 0x7fffffffffffffffLL;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      CT ov = __shfl_xor_sync(0xffffffffu, best, o);
      long long oi = __shfl_xor_sync(0xffffffffu, bi, o);
      comb(ov, oi);
    }
    if (lane == 0) y[blockIdx.x] = bi == 0x7fffffffffffffffLL ? 0 : bi;
  }
}

// Column reduction: CTA = 32 columns x 8 row lanes; grid (col tiles, splits, outer).
// With splits > 1 the result goes to part[outer][split][inner] (CT precision).
template <typename T, typename TO, int OP>
__global__ void col_reduce_kernel(const T* __restrict__ x, TO* __restrict__ y,
                                  typename Acc<T>::CT* __restrict__ part, long long R, long long inner,
                                  int splits, int to_part) {
  using CT = typename Acc<T>::CT;
  __shared__ CT sm[8][33];
  const long long col = (long long)blockIdx.x * 32 + threadIdx.x;
  const long long o = blockIdx.z;
  const long long per = (R + splits - 1) / splits;
  const long long r0 = (long long)blockIdx.y * per, r1 = min(r0 + per, R);
  CT a = r_init<CT, OP>();
  if (col < inner) {
    const T* xp = x + o * R * inner + col;
    for (long long r = r0 + threadIdx.y; r < r1; r += 8) a = r_comb<CT, OP>(a, (CT)xp[r * inner]);
  }
  sm[threadIdx.y][threadIdx.x] = a;
  __syncthreads();
  if (threadIdx.y == 0 && col < inner) {
#pragma unroll
    for (int k = 1; k < 8; k++) a = r_comb<CT, OP>(a, sm[k][threadIdx.x]);
    if (to_part) {
      if (GB_IN_BOUNDS(blockIdx.y, splits, 301)) part[(o * splits + blockIdx.y) * inner + col] = a;
    } else {
      if (OP == R_MEAN) a = a / (CT)R;
      y[o * inner + col] = (TO)a;
    }
  }
}

// Column reduction for 16-bit inputs whose row length is a multiple of 8: a thread owns 8
// adjacent columns and reads them as one 16-byte load; a CTA covers 256 columns x 8 row
// lanes with four rows in flight per thread.  Same outputs as col_reduce_kernel.
template <typename T, typename TO, int OP>
__global__ void __launch_bounds__(256)
col_reduce_vec_kernel(const T* __restrict__ x, TO* __restrict__ y, float* __restrict__ part, long long R,
                      long long inner, int splits, int to_part) {
  __shared__ float sm[8][8 * 32];
  const int tx = threadIdx.x, ty = threadIdx.y;
  const long long col0 = ((long long)blockIdx.x * 32 + tx) * 8;
  const long long o = blockIdx.z;
  const long long per = (R + splits - 1) / splits;
  const long long r0 = (long long)blockIdx.y * per, r1 = min(r0 + per, R);
  float a[8];
#pragma unroll
  for (int j = 0; j < 8; j++) a[j] = r_init<float, OP>();
  if (col0 < inner && GB_IN_BOUNDS(col0 + 7, inner, 303)) {   // a thread reads eight whole columns
    const T* xp = x + o * R * inner + col0;
    auto take = [&](const uint4& u) {
      const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
      for (int j = 0; j < 8; j++) a[j] = r_comb<float, OP>(a[j], (float)e[j]);
    };
    long long r = r0 + ty;
    // eight rows in flight per thread while there are that many, then four, then one
    for (; r + 56 < r1; r += 64) {
      const uint4 u0 = __ldg(reinterpret_cast<const uint4*>(xp + r * inner));
      const uint4 u1 = __ldg(reinterpret_cast<const uint4*>(xp + (r + 8) * inner));
      const uint4 u2 = __ldg(reinterpret_cast<const uint4*>(xp + (r + 16) * inner));
      const uint4 u3 = __ldg(reinterpret_cast<const uint4*>(xp + (r + 24) * inner));
      const uint4 u4 = __ldg(reinterpret_cast<const uint4*>(xp + (r + 32) * inner));
      const uint4 u5 = __ldg(reinterpret_cast<const uint4*>(xp + (r + 40) * inner));
      const uint4 u6 = __ldg(reinterpret_cast<const uint4*>(xp + (r + 48) * inner));
      const uint4 u7 = __ldg(reinterpret_cast<const uint4*>(xp + (r + 56) * inner));
      take(u0); take(u1); take(u2); take(u3); take(u4); take(u5); take(u6); take(u7);
    }
    for (; r + 24 < r1; r += 32) {
      const uint4 u0 = __ldg(reinterpret_cast<const uint4*>(xp + r * inner));
      const uint4 u1 = __ldg(reinterpret_cast<const uint4*>(xp + (r + 8) * inner));
      const uint4 u2 = __ldg(reinterpret_cast<const uint4*>(xp + (r + 16) * inner));
      const uint4 u3 = __ldg(reinterpret_cast<const uint4*>(xp + (r + 24) * inner));
      take(u0); take(u1); take(u2); take(u3);
    }
    for (; r < r1; r += 8) take(__ldg(reinterpret_cast<const uint4*>(xp + r * inner)));
  }
#pragma unroll
  for (int j = 0; j < 8; j++) sm[ty][j * 32 + tx] = a[j];
  __syncthreads();
  // thread (tx, ty) finishes column tx * 8 + ty of the CTA's 256
  const long long col = ((long long)blockIdx.x * 32 + tx) * 8 + ty;
  if (col < inner) {
    float v = sm[0][ty * 32 + tx];
#pragma unroll
    for (int k = 1; k < 8; k++) v = r_comb<float, OP>(v, sm[k][ty * 32 + tx]);
    if (to_part) {
      if (GB_IN_BOUNDS(blockIdx.y, splits, 302)) part[(o * splits + blockIdx.y) * inner + col] = v;
    } else {
      if (OP == R_MEAN) v = v / (float)R;
      y[o * inner + col] = (TO)v;
    }
  }
}

// Combines the per-split partial results: CTA = 32 columns x 8 split lanes, fixed order.
template <typename CT, typename TO, int OP>
__global__ void col_finish_kernel(const CT* __restrict__ part, TO* __restrict__ y, long long R,
                                  long long inner, int splits, long long outer, int accumulate) {
  __shared__ CT sm[8][33];
  const long long col = (long long)blockIdx.x * 32 + threadIdx.x;
  const long long o = blockIdx.y;
  CT a = r_init<CT, OP>();
  if (col < inner)
    for (int s = threadIdx.y; s < splits; s += 8) a = r_comb<CT, OP>(a, part[(o * splits + s) * inner + col]);
  sm[threadIdx.y][threadIdx.x] = a;
  __syncthreads();
  if (threadIdx.y == 0 && col < inner) {
#pragma unroll
    for (int k = 1; k < 8; k++) a = r_comb<CT, OP>(a, sm[k][threadIdx.x]);
    if (OP == R_MEAN) a = a / (CT)R;
    const long long i = o * inner + col;
    if (accumulate) a += (CT)y[i];
    y[i] = (TO)a;
  }
}

// Arg-max / arg-min over the rows of (outer, R, inner): CTA = 32 columns x 32 row lanes; a thread
// scans rows ty, ty + 32, ... of its column (consecutive threads read consecutive columns), then the
// 32 candidates of a column are combined in row-lane order.  Ties keep the smallest row index, the
// first occurrence, as a serial scan would.
template <typename T, int OP>
__global__ void __launch_bounds__(1024)
col_arg_kernel(const T* __restrict__ x, long long* __restrict__ y, long long R, long long inner) {
  using CT = typename Acc<T>::CT;
  __shared__ CT sv[32][33];
  __shared__ long long si[32][33];
  const long long col = (long long)blockIdx.x * 32 + threadIdx.x;
  const long long o = blockIdx.y;
  CT best = 0;
  long long bi = -1;
  if (col < inner) {
    const T* xp = x + o * R * inner + col;
    for (long long r = threadIdx.y; r < R; r += 32) {
      const CT v = (CT)xp[r * inner];
      if (bi < 0 || (OP == R_ARGMAX ? v > best : v < best)) { best = v; bi = r; }
    }
  }
  sv[threadIdx.y][threadIdx.x] = best;
  si[threadIdx.y][threadIdx.x] = bi;
  __syncthreads();
  if (threadIdx.y == 0 && col < inner) {
    for (int k = 1; k < 32; k++) {
      const CT v = sv[k][threadIdx.x];
      const long long r = si[k][threadIdx.x];
      if (r < 0) continue;
      const bool better = OP == R_ARGMAX ? v > best : v < best;
      if (bi < 0 || better || (v == best && r < bi)) { best = v; bi = r; }
    }
    y[o * inner + col] = bi < 0 ? 0 : bi;
  }
}

template <typename T, typename TO, int OP>
void launch_col_vec(dim3 grid, dim3 blk, cudaStream_t s, const void* x, void* y, void* scratch, long long R,
                    long long inner, int splits, int to_part) {
  if constexpr (sizeof(T) == 2) {
    col_reduce_vec_kernel<T, TO, OP><<<grid, blk, 0, s>>>((const T*)x, (TO*)y, (float*)scratch, R, inner, splits,
                                                          to_part);
  }
}

template <typename T, typename TO>
int reduce_t(int op, const void* x, void* y, void* scratch, long long scratch_bytes, long long outer,
             long long R, long long inner, int accumulate, cudaStream_t s) {
  using CT = typename Acc<T>::CT;
  if (outer <= 0 || inner <= 0 || R <= 0) return gbh::E_OK;
  if (op == R_ARGMAX || op == R_ARGMIN) {
    if (inner == 1) {
      int blk = R >= 1024 ? 256 : (R >= 128 ? 128 : 32);
      if (op == R_ARGMAX) row_arg_kernel<T, R_ARGMAX><<<(unsigned)outer, blk, 0, s>>>((const T*)x, (long long*)y, R);
      else row_arg_kernel<T, R_ARGMIN><<<(unsigned)outer, blk, 0, s>>>((const T*)x, (long long*)y, R);
    } else {
      if (outer > 65535) {
        gbh::set_error("reduce: arg-max over an inner axis supports at most 65535 outer slices");
        return gbh::E_TOO_LARGE;
      }
      const dim3 grid((unsigned)((inner + 31) / 32), (unsigned)outer), blk(32, 32);
      if (op == R_ARGMAX) col_arg_kernel<T, R_ARGMAX><<<grid, blk, 0, s>>>((const T*)x, (long long*)y, R, inner);
      else col_arg_kernel<T, R_ARGMIN><<<grid, blk, 0, s>>>((const T*)x, (long long*)y, R, inner);
    }
    GB_CUDA_OK(cudaGetLastError());
    return gbh::E_OK;
  }
#define GB_R(OPID)                                                                                   \
  case OPID:                                                                                         \
    if (inner == 1 && !accumulate) {                                                                 \
      int blk = R >= 4096 ? 512 : (R >= 512 ? 256 : (R >= 64 ? 64 : 32));                            \
      row_reduce_kernel<T, TO, OPID><<<(unsigned)outer, blk, 0, s>>>((const T*)x, (TO*)y, R);        \
    } else {                                                                                         \
      const bool vec = sizeof(T) == 2 && (inner & 7) == 0 && (((uintptr_t)x & 15) == 0);             \
      long long tiles = vec ? (inner + 255) / 256 : (inner + 31) / 32;                               \
      int splits = 1;                                                                                \
      if (tiles * outer < 148 * 4 && R >= 256) {                                                     \
        splits = (int)((148 * 4 + tiles * outer - 1) / (tiles * outer));                             \
        if (splits > R / 64) splits = (int)(R / 64);                                                 \
        if (splits < 1) splits = 1;                                                                  \
        while (splits > 1 && (long long)splits * outer * inner * (long long)sizeof(CT) > scratch_bytes) splits--; \
      }                                                                                              \
      const bool two = splits > 1 || accumulate;                                                     \
      if (two && (long long)splits * outer * inner * (long long)sizeof(CT) > scratch_bytes) {        \
        gbh::set_error("reduce: accumulate needs %lld bytes of scratch", (long long)splits * outer * inner * (long long)sizeof(CT)); \
        return gbh::E_BAD_ARG;                                                                       \
      }                                                                                              \
      dim3 grid((unsigned)tiles, splits, (unsigned)outer), blk(32, 8);                               \
      if (vec) launch_col_vec<T, TO, OPID>(grid, blk, s, x, y, scratch, R, inner, splits, two ? 1 : 0); \
      else col_reduce_kernel<T, TO, OPID><<<grid, blk, 0, s>>>((const T*)x, (TO*)y, (CT*)scratch, R, inner, splits, two ? 1 : 0); \
      if (two) {                                                                                     \
        dim3 fgrid((unsigned)((inner + 31) / 32), (unsigned)outer);                                  \
        col_finish_kernel<CT, TO, OPID><<<fgrid, dim3(32, 8), 0, s>>>((const CT*)scratch, (TO*)y, R, inner, splits, outer, accumulate); \
      }                                                                                              \
    }                                                                                                \
    break;
  switch (op) {
    GB_R(R_SUM) GB_R(R_MEAN) GB_R(R_MAX) GB_R(R_MIN)
    default:
      gbh::set_error("reduce: unknown op %d", op);
      return gbh::E_BAD_ARG;
  }
#undef GB_R
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

}  // namespace

enum { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2, DT_F64 = 3 };

// y[o, i] = reduce_r x[o, r, i].  op: 0 sum, 1 mean, 2 max, 3 min, 4 argmax,
// 5 argmin (y is int64).  out_dtype: the input dtype, or fp32 for 16-bit inputs.
// scratch (optional, scratch_bytes long) lets a column reduction split R across
// CTAs; accumulate adds the result onto y (sum / mean only, needs scratch).
GB_EXPORT int gb_reduce(int op, int dtype, int out_dtype, const void* x, void* y, void* scratch,
                        long long scratch_bytes, long long outer, long long R, long long inner,
                        int accumulate, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  GB_BOUNDS_BIND();
  if (scratch == nullptr) scratch_bytes = 0;
  if (dtype == DT_BF16 && out_dtype == DT_BF16) return reduce_t<__nv_bfloat16, __nv_bfloat16>(op, x, y, scratch, scratch_bytes, outer, R, inner, accumulate, s);
  if (dtype == DT_BF16 && out_dtype == DT_F32) return reduce_t<__nv_bfloat16, float>(op, x, y, scratch, scratch_bytes, outer, R, inner, accumulate, s);
  if (dtype == DT_F16 && out_dtype == DT_F16) return reduce_t<__half, __half>(op, x, y, scratch, scratch_bytes, outer, R, inner, accumulate, s);
  if (dtype == DT_F16 && out_dtype == DT_F32) return reduce_t<__half, float>(op, x, y, scratch, scratch_bytes, outer, R, inner, accumulate, s);
  if (dtype == DT_F32 && out_dtype == DT_F32) return reduce_t<float, float>(op, x, y, scratch, scratch_bytes, outer, R, inner, accumulate, s);
  if (dtype == DT_F64 && out_dtype == DT_F64) return reduce_t<double, double>(op, x, y, scratch, scratch_bytes, outer, R, inner, accumulate, s);
  gbh::set_error("gb_reduce: unsupported dtype pair %d -> %d", dtype, out_dtype);
  return gbh::E_BAD_ARG;
}
