// Sliding-window core shared by convolution, pooling, fold / unfold and padding.
//
// The reference builds, for every sliding-window layer, a dense 0/1 "gather
// matrix" G (numWin*winSize x prod(In)) and applies it with a GEMM
// (nn/gather.go:99-181, nn/conv.go:341-380, nn/pool.go:340-370).  Here the same
// information is an int32 index map idx[win][tap] (-1 = padding) and the gather
// is done by address: no multiply by zeros, no dense matrix.  The transpose of
// the gather (col2im, pooling backward) uses the inverted map in CSR form, so it
// is a gather too: deterministic, no atomics.
//
//   window_gather   col[n][win][c*T + tap] = x[n][c][idx[win][tap]]   (im2col; the row
//                   of one window is K-major for the GEMM that follows)
//   window_scatter  dx[n][c][i] = sum over (win,tap) with idx[win][tap]==i of
//                   dcol[n][win][c*T + tap]                              (col2im)
//   pool_fwd / pool_bwd   max (with argmax), average, LP-norm pooling over idx
#include "bounds.cuh"

using namespace gb;

namespace {

// q = i / d, r = i % d; 32-bit arithmetic when both operands fit (64-bit division costs
// tens of instructions and these kernels do one or two per element).
__device__ __forceinline__ void divmod(long long i, long long d, bool small, long long& q, long long& r) {
  if (small) {
    const unsigned ii = (unsigned)i, dd = (unsigned)d;
    const unsigned qq = ii / dd;
    q = qq;
    r = ii - qq * dd;
  } else {
    q = i / d;
    r = i - q * d;
  }
}

template <typename T>
__global__ void window_gather_kernel(const T* __restrict__ x, const int* __restrict__ idx,
                                     T* __restrict__ col, int N, int C, long long S, int nwin, int T_,
                                     int kpad, float fill) {
  // one thread per (n, win, k) with k = c*T + tap; k in [0, kpad), zero beyond C*T
  const long long total = (long long)N * nwin * kpad;
  const bool small = total <= 0x7fffffffLL;
  const int K = C * T_;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long r, kk, nn, ww;
    divmod(i, kpad, small, r, kk);
    divmod(r, nwin, small, nn, ww);
    const int k = (int)kk, win = (int)ww, n = (int)nn;
    T v = (T)0.f;
    if (k < K) {
      const int c = k / T_, tap = k - c * T_;
      const int src = idx[win * T_ + tap];
      v = (src >= 0 && GB_IN_BOUNDS(src, S, 101)) ? x[((long long)n * C + c) * S + src] : (T)fill;
    }
    col[i] = v;
  }
}

// dx[n][c][i] = sum_{e in csr(i)} dcol[n][win(e)][c*T + tap(e)], csr_cols[e] = win*T + tap
template <typename T>
__global__ void window_scatter_kernel(const T* __restrict__ dcol, const int* __restrict__ offs,
                                      const int* __restrict__ cols, T* __restrict__ dx, int N, int C,
                                      long long S, int nwin, int T_, int kpad, int accumulate) {
  const long long total = (long long)N * C * S;
  const bool small = total <= 0x7fffffffLL;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long pos, r, cc, nn;
    divmod(i, S, small, r, pos);
    divmod(r, C, small, nn, cc);
    const int c = (int)cc, n = (int)nn;
    float acc = 0.f;
    for (int e = offs[pos]; e < offs[pos + 1]; e++) {
      const int wt = cols[e];
      const int win = wt / T_, tap = wt - win * T_;
      if (!GB_IN_BOUNDS(wt, (long long)nwin * T_, 102)) continue;
      acc += (float)dcol[((long long)n * nwin + win) * kpad + c * T_ + tap];
    }
    dx[i] = accumulate ? (T)((float)dx[i] + acc) : (T)acc;
  }
}

enum PoolMode : int { POOL_MAX = 0, POOL_AVG = 1, POOL_LP = 2 };

// y[b][win] over taps idx[win][*]; b = n*C + c.  arg[b][win] = winning tap (max).
template <typename T>
__global__ void pool_fwd_kernel(const T* __restrict__ x, const int* __restrict__ idx,
                                T* __restrict__ y, int* __restrict__ arg, long long B, long long S,
                                int nwin, int T_, int mode, int count_include_pad, float p) {
  const long long total = B * nwin;
  const bool small = total <= 0x7fffffffLL && B * S <= 0x7fffffffLL;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long b, ww;
    divmod(i, nwin, small, b, ww);
    const int win = (int)ww;
    const T* xb = x + b * S;
    const int* iw = idx + (long long)win * T_;
    if (mode == POOL_MAX) {
      float best = -INFINITY;
      int bt = -1;
      for (int t = 0; t < T_; t++) {
        const int src = iw[t];
        if (src < 0 || !GB_IN_BOUNDS(src, S, 103)) continue;
        const float v = (float)xb[src];
        if (v > best || bt < 0) { best = v; bt = t; }
      }
      y[i] = (T)(bt < 0 ? 0.f : best);
      if (arg) arg[i] = bt;
    } else if (mode == POOL_AVG) {
      float s = 0.f;
      int cnt = 0;
      for (int t = 0; t < T_; t++) {
        const int src = iw[t];
        if (src >= 0 && GB_IN_BOUNDS(src, S, 104)) { s += (float)xb[src]; cnt++; }
      }
      const int div = count_include_pad ? T_ : (cnt > 0 ? cnt : 1);
      y[i] = (T)(s / (float)div);
    } else {
      float s = 0.f;
      for (int t = 0; t < T_; t++) {
        const int src = iw[t];
        if (src >= 0 && GB_IN_BOUNDS(src, S, 105)) s += powf((float)xb[src], p);
      }
      y[i] = (T)powf(s, 1.f / p);
    }
  }
}

// Max / average pooling with at most 8 taps per window (2 x 2, 2 x 2 x 2, ...): a thread keeps the
// tap offsets of its windows in registers and walks the planes of its blockIdx.y slice, so the index
// map is read once per thread instead of once per output.
template <typename T>
__global__ void pool_fwd_small_kernel(const T* __restrict__ x, const int* __restrict__ idx, T* __restrict__ y,
                                      int* __restrict__ arg, long long B, long long S, int nwin, int T_, int mode,
                                      int count_include_pad) {
  for (int win = blockIdx.x * blockDim.x + threadIdx.x; win < nwin; win += gridDim.x * blockDim.x) {
    int src[8];
    int cnt = 0;
#pragma unroll
    for (int t = 0; t < 8; t++) {
      src[t] = t < T_ ? __ldg(idx + (long long)win * T_ + t) : -1;
      if (src[t] >= 0 && !GB_IN_BOUNDS(src[t], S, 108)) src[t] = -1;
      cnt += src[t] >= 0;
    }
    const float inv = 1.f / (float)(count_include_pad ? T_ : (cnt > 0 ? cnt : 1));
#pragma unroll 4
    for (long long b = blockIdx.y; b < B; b += gridDim.y) {
      const T* xb = x + b * S;
      float v[8];
#pragma unroll
      for (int t = 0; t < 8; t++) v[t] = src[t] >= 0 ? (float)xb[src[t]] : 0.f;
      if (mode == POOL_MAX) {
        float best = 0.f;
        int bt = -1;
#pragma unroll
        for (int t = 0; t < 8; t++)
          if (src[t] >= 0 && (v[t] > best || bt < 0)) { best = v[t]; bt = t; }
        y[b * nwin + win] = (T)best;
        if (arg) arg[b * nwin + win] = bt;
      } else {
        float sum = 0.f;
#pragma unroll
        for (int t = 0; t < 8; t++) sum += v[t];
        y[b * nwin + win] = (T)(sum * inv);
      }
    }
  }
}

// Max / average pooling over wide windows (global pooling: one window of H * W taps): one warp per
// output, lanes along the taps, then a shuffle reduction.  The arg-max is the first tap that holds the
// maximum, as in the one-thread-per-output kernel.
template <typename T>
__global__ void pool_fwd_wide_kernel(const T* __restrict__ x, const int* __restrict__ idx, T* __restrict__ y,
                                     int* __restrict__ arg, long long B, long long S, int nwin, int T_, int mode,
                                     int count_include_pad) {
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const long long total = B * nwin;
  for (long long o = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); o < total; o += (long long)gridDim.x * wpb) {
    const long long b = o / nwin;
    const int win = (int)(o - b * nwin);
    const T* xb = x + b * S;
    const int* iw = idx + (long long)win * T_;
    float best = -INFINITY, sum = 0.f;
    int bt = 0x7fffffff, cnt = 0;
    for (int t = lane; t < T_; t += 32) {
      const int src = __ldg(iw + t);
      if (src < 0 || !GB_IN_BOUNDS(src, S, 109)) continue;
      const float v = (float)xb[src];
      sum += v;
      cnt++;
      if (v > best || bt == 0x7fffffff) { best = v; bt = t; }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, off);
      const int ot = __shfl_xor_sync(0xffffffffu, bt, off);
      sum += __shfl_xor_sync(0xffffffffu, sum, off);
      cnt += __shfl_xor_sync(0xffffffffu, cnt, off);
      // a lane that saw no tap holds (-inf, INT_MAX) and always loses; equal values keep the earlier tap
      if (ot != 0x7fffffff && (bt == 0x7fffffff || ov > best || (ov == best && ot < bt))) { best = ov; bt = ot; }
    }
    if (lane == 0) {
      if (mode == POOL_MAX) {
        y[o] = (T)(bt == 0x7fffffff ? 0.f : best);
        if (arg) arg[o] = bt == 0x7fffffff ? -1 : bt;
      } else {
        y[o] = (T)(sum / (float)(count_include_pad ? T_ : (cnt > 0 ? cnt : 1)));
      }
    }
  }
}

// dx[b][i] = sum over (win,tap) covering i of the window's gradient share
template <typename T>
__global__ void pool_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                const T* __restrict__ y, const int* __restrict__ arg,
                                const int* __restrict__ idx, const int* __restrict__ offs,
                                const int* __restrict__ cols, T* __restrict__ dx, long long B,
                                long long S, int nwin, int T_, int mode, int count_include_pad,
                                float p) {
  const long long total = B * S;
  const bool small = total <= 0x7fffffffLL;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long pos, b;
    divmod(i, S, small, b, pos);
    float acc = 0.f;
    for (int e = offs[pos]; e < offs[pos + 1]; e++) {
      const int wt = cols[e];
      const int win = wt / T_, tap = wt - win * T_;
      if (!GB_IN_BOUNDS(wt, (long long)nwin * T_, 106)) continue;
      const long long o = b * nwin + win;
      if (mode == POOL_MAX) {
        if (arg[o] == tap) acc += (float)dy[o];
      } else if (mode == POOL_AVG) {
        int div = T_;
        if (!count_include_pad) {
          int cnt = 0;
          for (int t = 0; t < T_; t++) cnt += idx[(long long)win * T_ + t] >= 0;
          div = cnt > 0 ? cnt : 1;
        }
        acc += (float)dy[o] / (float)div;
      } else {
        // d/dx (sum x^p)^(1/p) = x^(p-1) * y^(1-p)
        const float yv = (float)y[o];
        if (yv != 0.f) acc += (float)dy[o] * powf((float)x[i], p - 1.f) * powf(yv, 1.f - p);
      }
    }
    dx[i] = (T)acc;
  }
}

// Backward of max / average pooling whose windows do not overlap (every input position lies in at
// most one window: the usual stride == kernel case and global pooling).  p2w[pos] = {window, tap}
// of the position, or {-1, 0}; wcnt[win] = taps of the window that are not padding.  One thread
// per input element, rows (b) along blockIdx.y: no division, one table read and two dependent
// loads per element, coalesced stores.
template <typename T>
__global__ void pool_bwd_disjoint_kernel(const T* __restrict__ dy, const int* __restrict__ arg,
                                         const int2* __restrict__ p2w, const int* __restrict__ wcnt,
                                         T* __restrict__ dx, long long B, int S, int nwin, int T_, int mode,
                                         int count_include_pad) {
  // A thread keeps its positions' table entries in registers and walks the planes (b) of its
  // blockIdx.y slice, four at a time so that their loads are in flight together.
  for (int pos = blockIdx.x * blockDim.x + threadIdx.x; pos < S; pos += gridDim.x * blockDim.x) {
    const int2 w = __ldg(p2w + pos);
    const bool hit = w.x >= 0 && GB_IN_BOUNDS(w.x, nwin, 107);
    float inv = 1.f;
    if (hit && mode != POOL_MAX) inv = 1.f / (float)(count_include_pad ? T_ : max(__ldg(wcnt + w.x), 1));
    long long b = blockIdx.y;
    const long long step = gridDim.y;
    for (; b + 3 * step < B; b += 4 * step) {
      float g[4];
      int a4[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const long long bb = b + u * step;
        g[u] = hit ? (float)dy[bb * nwin + w.x] : 0.f;
        a4[u] = (hit && mode == POOL_MAX) ? arg[bb * nwin + w.x] : w.y;
      }
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const float v = mode == POOL_MAX ? (a4[u] == w.y ? g[u] : 0.f) : g[u] * inv;
        dx[(b + u * step) * S + pos] = (T)(hit ? v : 0.f);
      }
    }
    for (; b < B; b += step) {
      float v = 0.f;
      if (hit) {
        const float g = (float)dy[b * nwin + w.x];
        v = mode == POOL_MAX ? (arg[b * nwin + w.x] == w.y ? g : 0.f) : g * inv;
      }
      dx[b * S + pos] = (T)v;
    }
  }
}

inline int grid_for(long long work) {
  long long g = (work + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  if (g < 1) g = 1;
  return (int)g;
}

}  // namespace

enum { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2, DT_F64 = 3 };

#define GB_DISPATCH_T(CALL)                                   \
  switch (dtype) {                                            \
    case DT_BF16: { using T = __nv_bfloat16; CALL; } break;   \
    case DT_F16: { using T = __half; CALL; } break;           \
    case DT_F32: { using T = float; CALL; } break;            \
    default:                                                  \
      gbh::set_error("window op: unsupported dtype %d", dtype); \
      return gbh::E_BAD_ARG;                                  \
  }

// im2col: x (N,C,S) -> col (N, nwin, kpad) with K = C*T real columns (zero padded to kpad)
GB_EXPORT int gb_window_gather(int dtype, const void* x, const int* idx, void* col, int N, int C,
                               long long S, int nwin, int T_, int kpad, float fill, void* stream) {
  const long long total = (long long)N * nwin * kpad;
  if (total <= 0) return gbh::E_OK;
  cudaStream_t s = (cudaStream_t)stream;
  GB_BOUNDS_BIND();
  GB_DISPATCH_T((window_gather_kernel<T><<<grid_for(total), 256, 0, s>>>((const T*)x, idx, (T*)col, N, C, S, nwin, T_, kpad, fill)));
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

// col2im: dcol (N, nwin, kpad) -> dx (N,C,S) through the inverted index map (CSR over S)
GB_EXPORT int gb_window_scatter(int dtype, const void* dcol, const int* offs, const int* cols,
                                void* dx, int N, int C, long long S, int nwin, int T_, int kpad,
                                int accumulate, void* stream) {
  const long long total = (long long)N * C * S;
  if (total <= 0) return gbh::E_OK;
  cudaStream_t s = (cudaStream_t)stream;
  GB_BOUNDS_BIND();
  GB_DISPATCH_T((window_scatter_kernel<T><<<grid_for(total), 256, 0, s>>>((const T*)dcol, offs, cols, (T*)dx, N, C, S, nwin, T_, kpad, accumulate)));
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

// mode: 0 max (arg receives the winning tap per window, may be null), 1 average, 2 LP norm
GB_EXPORT int gb_pool_fwd(int dtype, const void* x, const int* idx, void* y, int* arg, long long B,
                          long long S, int nwin, int T_, int mode, int count_include_pad, float p,
                          void* stream) {
  const long long total = B * nwin;
  if (total <= 0) return gbh::E_OK;
  cudaStream_t s = (cudaStream_t)stream;
  GB_BOUNDS_BIND();
  if (mode != POOL_LP && T_ <= 8 && B >= 64) {
    const int bx = (nwin + 255) / 256 < 64 ? (nwin + 255) / 256 : 64;
    long long by = (148 * 8 + bx - 1) / bx;
    if (by > B) by = B;
    GB_DISPATCH_T((pool_fwd_small_kernel<T><<<dim3(bx, (unsigned)by), 256, 0, s>>>((const T*)x, idx, (T*)y, arg, B, S, nwin, T_, mode, count_include_pad)));
    GB_CUDA_OK(cudaGetLastError());
    return gbh::E_OK;
  }
  if (mode != POOL_LP && T_ >= 64) {
    const long long warps = total;
    const int grid = (int)((warps + 7) / 8 < 148 * 8 ? (warps + 7) / 8 : 148 * 8);
    GB_DISPATCH_T((pool_fwd_wide_kernel<T><<<grid, 256, 0, s>>>((const T*)x, idx, (T*)y, arg, B, S, nwin, T_, mode, count_include_pad)));
    GB_CUDA_OK(cudaGetLastError());
    return gbh::E_OK;
  }
  GB_DISPATCH_T((pool_fwd_kernel<T><<<grid_for(total), 256, 0, s>>>((const T*)x, idx, (T*)y, arg, B, S, nwin, T_, mode, count_include_pad, p)));
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

// Backward for non-overlapping windows (max or average): see pool_bwd_disjoint_kernel.
GB_EXPORT int gb_pool_bwd_disjoint(int dtype, const void* dy, const int* arg, const int* p2w, const int* wcnt,
                                   void* dx, long long B, long long S, int nwin, int T_, int mode,
                                   int count_include_pad, void* stream) {
  if (B <= 0 || S <= 0) return gbh::E_OK;
  if (mode != POOL_MAX && mode != POOL_AVG) {
    gbh::set_error("gb_pool_bwd_disjoint: max or average pooling only");
    return gbh::E_BAD_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  GB_BOUNDS_BIND();
  const int bx = (int)((S + 255) / 256 < 64 ? (S + 255) / 256 : 64);
  // about eight CTAs per SM in total; every CTA walks B / by planes
  long long by = (148 * 8 + bx - 1) / bx;
  if (by > B) by = B;
  if (by < 1) by = 1;
  GB_DISPATCH_T((pool_bwd_disjoint_kernel<T><<<dim3(bx, (unsigned)by), 256, 0, s>>>((const T*)dy, arg, (const int2*)p2w, wcnt, (T*)dx, B, (int)S, nwin, T_, mode, count_include_pad)));
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

GB_EXPORT int gb_pool_bwd(int dtype, const void* dy, const void* x, const void* y, const int* arg,
                          const int* idx, const int* offs, const int* cols, void* dx, long long B,
                          long long S, int nwin, int T_, int mode, int count_include_pad, float p,
                          void* stream) {
  const long long total = B * S;
  if (total <= 0) return gbh::E_OK;
  cudaStream_t s = (cudaStream_t)stream;
  GB_BOUNDS_BIND();
  GB_DISPATCH_T((pool_bwd_kernel<T><<<grid_for(total), 256, 0, s>>>((const T*)dy, (const T*)x, (const T*)y, arg, idx, offs, cols, (T*)dx, B, S, nwin, T_, mode, count_include_pad, p)));
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}
