// Row softmax / log-softmax (forward and backward) and fused cross-entropy
// (forward: per-row loss and log-sum-exp; backward: dlogits, optionally written
// over the logits).  One CTA per row; the row is staged once in shared memory
// (in its storage dtype) when it fits, so global memory is read once.
//
// The reference composes Softmax/LogSoftmax from six tape nodes
// (tensor/ops_activation.go:454-470) and CrossEntropyLoss from LogSoftmax +
// Gather with class weights, ignore index and label smoothing
// (nn/loss.go:131-242); the mean reduction divides by the summed weights of the
// non-ignored targets.
#include "common.cuh"

using namespace gb;

namespace {

constexpr int kMaxStageBytes = 200 * 1024;

template <typename T> __device__ __forceinline__ float ldf(const T* p, long long i) { return (float)p[i]; }

// Copies a row into shared memory (vectorised when aligned) or leaves it in
// global memory; returns the pointer to read from.
template <typename T>
__device__ __forceinline__ const T* stage_row(const T* __restrict__ g, T* sm, int D, bool use_smem) {
  if (!use_smem) return g;
  constexpr int V = 16 / sizeof(T);
  if ((((uintptr_t)g) & 15) == 0) {
    const int nv = D / V;
    const uint4* gv = reinterpret_cast<const uint4*>(g);
    uint4* sv = reinterpret_cast<uint4*>(sm);
    for (int i = threadIdx.x; i < nv; i += blockDim.x) sv[i] = gv[i];
    for (int i = nv * V + threadIdx.x; i < D; i += blockDim.x) sm[i] = g[i];
  } else {
    for (int i = threadIdx.x; i < D; i += blockDim.x) sm[i] = g[i];
  }
  __syncthreads();
  return sm;
}

// MODE 0: softmax, 1: log_softmax
template <typename T, int MODE>
__global__ void softmax_fwd_kernel(const T* __restrict__ x, T* __restrict__ y, int D, int use_smem) {
  extern __shared__ __align__(16) unsigned char smraw[];
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const T* xr = stage_row<T>(x + row * D, (T*)smraw, D, use_smem);
  float m = -INFINITY;
  for (int i = threadIdx.x; i < D; i += blockDim.x) m = fmaxf(m, (float)xr[i]);
  m = block_max(m, red);
  float s = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) s += __expf((float)xr[i] - m);
  s = block_sum(s, red);
  const float inv = 1.f / s, ls = logf(s);
  T* yr = y + row * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float v = (float)xr[i] - m;
    yr[i] = (T)(MODE == 0 ? __expf(v) * inv : v - ls);
  }
}

// MODE 0: dx = y * (dy - sum(dy*y));  MODE 1: dx = dy - exp(y) * sum(dy)
template <typename T, int MODE>
__global__ void softmax_bwd_kernel(const T* __restrict__ y, const T* __restrict__ dy,
                                   T* __restrict__ dx, int D) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const T* yr = y + row * D;
  const T* gr = dy + row * D;
  float s = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x)
    s += MODE == 0 ? (float)gr[i] * (float)yr[i] : (float)gr[i];
  s = block_sum(s, red);
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float yv = (float)yr[i], g = (float)gr[i];
    dx[row * D + i] = (T)(MODE == 0 ? yv * (g - s) : g - __expf(yv) * s);
  }
}

// Softmax / log-softmax for 16-bit rows whose length is a multiple of 8: one pass over the row with
// 16-byte loads and a running (max, sum) pair per thread, then a second pass (served by the cache) that
// writes 16 bytes at a time.  No shared-memory copy of the row.
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
softmax_fwd_vec_kernel(const T* __restrict__ x, T* __restrict__ y, int D) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * D);
  uint4* yr = reinterpret_cast<uint4*>(y + row * D);
  const int nvec = D / 8;
  float m = -INFINITY, s = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 u = xr[v];
    const T* e = reinterpret_cast<const T*>(&u);
    float f[8], mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; j++) { f[j] = (float)e[j]; mx = fmaxf(mx, f[j]); }
    if (mx > m) { s *= __expf(m - mx); m = mx; }
#pragma unroll
    for (int j = 0; j < 8; j++) s += __expf(f[j] - m);
  }
  const float M = block_max(m, red);
  s = block_sum(m == -INFINITY ? 0.f : s * __expf(m - M), red);
  const float inv = 1.f / s, ls = logf(s);
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 u = xr[v];
    const T* e = reinterpret_cast<const T*>(&u);
    alignas(16) T o[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const float d = (float)e[j] - M;
      o[j] = (T)(MODE == 0 ? __expf(d) * inv : d - ls);
    }
    yr[v] = *reinterpret_cast<const uint4*>(o);
  }
}

template <typename T, int MODE>
__global__ void __launch_bounds__(256)
softmax_bwd_vec_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx, int D) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const uint4* yr = reinterpret_cast<const uint4*>(y + row * D);
  const uint4* gr = reinterpret_cast<const uint4*>(dy + row * D);
  uint4* dr = reinterpret_cast<uint4*>(dx + row * D);
  const int nvec = D / 8;
  float s = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 a = yr[v], b = gr[v];
    const T* ya = reinterpret_cast<const T*>(&a);
    const T* gb_ = reinterpret_cast<const T*>(&b);
#pragma unroll
    for (int j = 0; j < 8; j++) s += MODE == 0 ? (float)gb_[j] * (float)ya[j] : (float)gb_[j];
  }
  s = block_sum(s, red);
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 a = yr[v], b = gr[v];
    const T* ya = reinterpret_cast<const T*>(&a);
    const T* gb_ = reinterpret_cast<const T*>(&b);
    alignas(16) T o[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const float yv = (float)ya[j], g = (float)gb_[j];
      o[j] = (T)(MODE == 0 ? yv * (g - s) : g - __expf(yv) * s);
    }
    dr[v] = *reinterpret_cast<const uint4*>(o);
  }
}

// Cross-entropy forward.  Per row: lse, weighted loss (0 for ignored rows) and
// the effective weight (the row's contribution to the mean denominator).
template <typename T>
__global__ void ce_fwd_kernel(const T* __restrict__ x, const long long* __restrict__ tgt,
                              const float* __restrict__ cw, float* __restrict__ loss_row,
                              float* __restrict__ lse_out, float* __restrict__ w_row, int C,
                              long long ignore_index, int has_ignore, float eps, float cw_sum,
                              int use_smem, int* status) {
  extern __shared__ __align__(16) unsigned char smraw[];
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const T* xr = stage_row<T>(x + row * C, (T*)smraw, C, use_smem);
  float m = -INFINITY;
  for (int i = threadIdx.x; i < C; i += blockDim.x) m = fmaxf(m, (float)xr[i]);
  m = block_max(m, red);
  float s = 0.f, sx = 0.f;
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    float v = (float)xr[i];
    s += __expf(v - m);
    if (eps != 0.f) sx += (cw ? cw[i] : 1.f) * v;
  }
  s = block_sum(s, red);
  if (eps != 0.f) sx = block_sum(sx, red);
  if (threadIdx.x == 0) {
    const float lse = m + logf(s);
    lse_out[row] = lse;
    long long t = tgt[row];
    float loss = 0.f, w = 0.f;
    const bool ignored = has_ignore && t == ignore_index;
    if (!ignored) {
      if (t < 0 || t >= C) {
        set_status(status, ST_BAD_INDEX, (int)row);
      } else {
        w = cw ? cw[t] : 1.f;
        loss = (1.f - eps) * w * (lse - (float)xr[t]);
        // smoothing term: (eps / C) * sum_c w_c * (lse - x_c)
        if (eps != 0.f) loss += (eps / C) * (cw_sum * lse - sx);
      }
    }
    loss_row[row] = loss;
    w_row[row] = w;
  }
}

// The same for 16-bit logits without label smoothing and a class count that is a multiple
// of 8: one pass over global memory with 16-byte loads and a running (max, sum) pair per
// thread, combined across the CTA at the end.  No shared-memory copy of the row.
template <typename T>
__global__ void __launch_bounds__(256)
ce_fwd_vec_kernel(const T* __restrict__ x, const long long* __restrict__ tgt, const float* __restrict__ cw,
                  float* __restrict__ loss_row, float* __restrict__ lse_out, float* __restrict__ w_row, int C,
                  long long ignore_index, int has_ignore, int* status) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * C);
  const int nvec = C / 8;
  float m = -INFINITY, s = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 u = __ldg(xr + v);
    const T* e = reinterpret_cast<const T*>(&u);
    float f[8];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; j++) { f[j] = (float)e[j]; mx = fmaxf(mx, f[j]); }
    if (mx > m) {
      s *= __expf(m - mx);  // exp(-inf) = 0 on the first vector
      m = mx;
    }
#pragma unroll
    for (int j = 0; j < 8; j++) s += __expf(f[j] - m);
  }
  const float M = block_max(m, red);
  s = block_sum(m == -INFINITY ? 0.f : s * __expf(m - M), red);
  if (threadIdx.x == 0) {
    const float lse = M + logf(s);
    lse_out[row] = lse;
    const long long t = tgt[row];
    float loss = 0.f, w = 0.f;
    const bool ignored = has_ignore && t == ignore_index;
    if (!ignored) {
      if (t < 0 || t >= C) {
        set_status(status, ST_BAD_INDEX, (int)row);
      } else {
        w = cw ? cw[t] : 1.f;
        loss = w * (lse - (float)x[row * C + t]);
      }
    }
    loss_row[row] = loss;
    w_row[row] = w;
  }
}

// Forward and gradient in one kernel, for a loss that is the root of the backward pass: the row is
// read once from memory (the second pass over it hits the cache), the loss terms are written as in
// ce_fwd_vec_kernel, and scale * (softmax - onehot) replaces the logits in place.  16-bit logits,
// class count a multiple of 8, no class weights, no ignored index, no label smoothing; scale is
// 1 / rows for the mean and 1 for the sum.  The reference computes the same two quantities as
// separate tape nodes (nn/loss.go CrossEntropyLoss: log-softmax, gather, mean).
template <typename T>
__global__ void __launch_bounds__(256)
ce_fused_vec_kernel(T* x, const long long* __restrict__ tgt, float* __restrict__ loss_row,
                    float* __restrict__ w_row, int C, float scale, int* status) {
  __shared__ float red[32];
  __shared__ float s_lse;
  const long long row = blockIdx.x;
  uint4* xr = reinterpret_cast<uint4*>(x + row * C);
  const int nvec = C / 8;
  float m = -INFINITY, s = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 u = xr[v];
    const T* e = reinterpret_cast<const T*>(&u);
    float f[8];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; j++) { f[j] = (float)e[j]; mx = fmaxf(mx, f[j]); }
    if (mx > m) {
      s *= __expf(m - mx);
      m = mx;
    }
#pragma unroll
    for (int j = 0; j < 8; j++) s += __expf(f[j] - m);
  }
  const float M = block_max(m, red);
  s = block_sum(m == -INFINITY ? 0.f : s * __expf(m - M), red);
  long long t = tgt[row];
  const bool bad = t < 0 || t >= C;
  if (threadIdx.x == 0) {
    const float lse = M + logf(s);
    s_lse = lse;
    if (bad) set_status(status, ST_BAD_INDEX, (int)row);
    loss_row[row] = bad ? 0.f : lse - (float)x[row * C + t];   // read before any thread overwrites the row
    w_row[row] = bad ? 0.f : 1.f;
  }
  __syncthreads();
  const float lse = s_lse;
  const float g = bad ? 0.f : scale;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 u = xr[v];
    const T* e = reinterpret_cast<const T*>(&u);
    alignas(16) T o[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      float d = g * __expf((float)e[j] - lse);
      if ((long long)v * 8 + j == t) d -= g;
      o[j] = (T)d;
    }
    xr[v] = *reinterpret_cast<const uint4*>(o);
  }
}

// x *= g[0] unless g[0] is exactly 1 (the usual case: the loss is the root of the backward pass),
// in which case every CTA returns after reading the scalar.
template <typename T>
__global__ void scale_unless_one_kernel(T* x, long long nvec, const float* __restrict__ g) {
  const float gv = g[0];
  if (gv == 1.f) return;
  uint4* xv = reinterpret_cast<uint4*>(x);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    uint4 u = xv[i];
    T* e = reinterpret_cast<T*>(&u);
#pragma unroll
    for (int j = 0; j < 8; j++) e[j] = (T)((float)e[j] * gv);
    xv[i] = u;
  }
}

// Sums loss_row and w_row (single CTA, fixed order per thread then tree) and
// writes out[0] = total loss (mean: / denom), out[1] = denom.
__global__ void ce_reduce_kernel(const float* __restrict__ loss_row, const float* __restrict__ w_row,
                                 long long rows, int mean, float* __restrict__ out) {
  __shared__ float red[32];
  float a = 0.f, b = 0.f;
  for (long long i = threadIdx.x; i < rows; i += blockDim.x) { a += loss_row[i]; b += w_row[i]; }
  a = block_sum(a, red);
  b = block_sum(b, red);
  if (threadIdx.x == 0) {
    out[0] = mean ? a / b : a;
    out[1] = b;
  }
}

// Cross-entropy backward: dlogits may alias the logits.
//   d/dx_c = g_row * [ ((1-eps) w_y + (eps/C) W) p_c - (1-eps) w_y [c==y] - (eps/C) w_c ]
// g_row = gscalar[0] (/ denom for mean) or grow[row] for reduction 'none'.
template <typename T>
__global__ void ce_bwd_kernel(const T* x, const long long* __restrict__ tgt,
                              const float* __restrict__ cw, const float* __restrict__ lse_in,
                              const float* __restrict__ gscalar, const float* __restrict__ grow,
                              const float* __restrict__ denom, T* dx, int C, long long ignore_index,
                              int has_ignore, float eps, float cw_sum) {
  const long long row = blockIdx.x;
  const long long t = tgt[row];
  const bool ignored = (has_ignore && t == ignore_index) || t < 0 || t >= C;
  T* dr = dx + row * C;
  if (ignored) {
    for (int i = threadIdx.x; i < C; i += blockDim.x) dr[i] = (T)0.f;
    return;
  }
  float g = grow ? grow[row] : gscalar[0];
  if (denom) g /= denom[0];
  const float wy = cw ? cw[t] : 1.f;
  const float lse = lse_in[row];
  const float a = g * ((1.f - eps) * wy + (eps / C) * cw_sum);
  const float hit = g * (1.f - eps) * wy;
  const float sm = g * (eps / C);
  const T* xr = x + row * C;
  constexpr int V = 16 / sizeof(T);
  if (eps == 0.f && (C % V) == 0 && ((((uintptr_t)xr | (uintptr_t)dr)) & 15) == 0) {
    struct alignas(16) Pack { T v[V]; };
    const Pack* xv = reinterpret_cast<const Pack*>(xr);
    Pack* dv = reinterpret_cast<Pack*>(dr);
    for (int i = threadIdx.x; i < C / V; i += blockDim.x) {
      Pack p = xv[i], o;
#pragma unroll
      for (int j = 0; j < V; j++) {
        float v = a * __expf((float)p.v[j] - lse);
        if ((long long)i * V + j == t) v -= hit;
        o.v[j] = (T)v;
      }
      dv[i] = o;
    }
    return;
  }
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    float v = a * __expf((float)xr[i] - lse);
    if (i == t) v -= hit;
    if (eps != 0.f) v -= sm * (cw ? cw[i] : 1.f);
    dr[i] = (T)v;
  }
}

inline int block_for(int D) {
  int b = 32;
  while (b < 512 && b * 8 < D) b <<= 1;
  return b;
}

template <typename T>
int set_smem(const void* kern, int D, int* use_smem, size_t* bytes) {
  size_t need = (size_t)D * sizeof(T);
  need = (need + 15) & ~(size_t)15;
  if (need <= (size_t)kMaxStageBytes) {
    *use_smem = 1;
    *bytes = need;
    if (need > 48 * 1024)
      GB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need));
  } else {
    *use_smem = 0;
    *bytes = 0;
  }
  return gbh::E_OK;
}

template <typename T>
int softmax_fwd_t(int mode, const void* x, void* y, long long rows, int D, cudaStream_t s) {
  if constexpr (sizeof(T) == 2) {
    if ((D & 7) == 0 && D >= 256 && ((((uintptr_t)x | (uintptr_t)y) & 15) == 0)) {
      if (mode) softmax_fwd_vec_kernel<T, 1><<<(unsigned)rows, 256, 0, s>>>((const T*)x, (T*)y, D);
      else softmax_fwd_vec_kernel<T, 0><<<(unsigned)rows, 256, 0, s>>>((const T*)x, (T*)y, D);
      GB_CUDA_OK(cudaGetLastError());
      return gbh::E_OK;
    }
  }
  int use_smem;
  size_t bytes;
  const void* k = mode ? (const void*)softmax_fwd_kernel<T, 1> : (const void*)softmax_fwd_kernel<T, 0>;
  int rc = set_smem<T>(k, D, &use_smem, &bytes);
  if (rc) return rc;
  if (mode) softmax_fwd_kernel<T, 1><<<(unsigned)rows, block_for(D), bytes, s>>>((const T*)x, (T*)y, D, use_smem);
  else softmax_fwd_kernel<T, 0><<<(unsigned)rows, block_for(D), bytes, s>>>((const T*)x, (T*)y, D, use_smem);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

template <typename T>
int softmax_bwd_t(int mode, const void* y, const void* dy, void* dx, long long rows, int D, cudaStream_t s) {
  if constexpr (sizeof(T) == 2) {
    if ((D & 7) == 0 && D >= 256 && ((((uintptr_t)y | (uintptr_t)dy | (uintptr_t)dx) & 15) == 0)) {
      if (mode) softmax_bwd_vec_kernel<T, 1><<<(unsigned)rows, 256, 0, s>>>((const T*)y, (const T*)dy, (T*)dx, D);
      else softmax_bwd_vec_kernel<T, 0><<<(unsigned)rows, 256, 0, s>>>((const T*)y, (const T*)dy, (T*)dx, D);
      GB_CUDA_OK(cudaGetLastError());
      return gbh::E_OK;
    }
  }
  if (mode) softmax_bwd_kernel<T, 1><<<(unsigned)rows, block_for(D), 0, s>>>((const T*)y, (const T*)dy, (T*)dx, D);
  else softmax_bwd_kernel<T, 0><<<(unsigned)rows, block_for(D), 0, s>>>((const T*)y, (const T*)dy, (T*)dx, D);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

template <typename T>
int ce_fwd_t(const void* x, const long long* tgt, const float* cw, float* loss_row, float* lse,
             float* w_row, long long rows, int C, long long ignore_index, int has_ignore, float eps,
             float cw_sum, cudaStream_t s) {
  if constexpr (sizeof(T) == 2) {
    if (eps == 0.f && (C & 7) == 0 && (((uintptr_t)x & 15) == 0)) {
      ce_fwd_vec_kernel<T><<<(unsigned)rows, 256, 0, s>>>((const T*)x, tgt, cw, loss_row, lse, w_row, C,
                                                          ignore_index, has_ignore, gbh::status_ptr());
      GB_CUDA_OK(cudaGetLastError());
      return gbh::E_OK;
    }
  }
  int use_smem;
  size_t bytes;
  int rc = set_smem<T>((const void*)ce_fwd_kernel<T>, C, &use_smem, &bytes);
  if (rc) return rc;
  ce_fwd_kernel<T><<<(unsigned)rows, block_for(C), bytes, s>>>((const T*)x, tgt, cw, loss_row, lse, w_row, C,
                                                              ignore_index, has_ignore, eps, cw_sum,
                                                              use_smem, gbh::status_ptr());
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

}  // namespace

enum { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2, DT_F64 = 3 };

// mode 0 = softmax, 1 = log_softmax over the last dimension of a (rows, D) tensor
GB_EXPORT int gb_softmax_fwd(int mode, int dtype, const void* x, void* y, long long rows, int D,
                             void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (rows <= 0 || D <= 0) return gbh::E_OK;
  switch (dtype) {
    case DT_BF16: return softmax_fwd_t<__nv_bfloat16>(mode, x, y, rows, D, s);
    case DT_F16: return softmax_fwd_t<__half>(mode, x, y, rows, D, s);
    case DT_F32: return softmax_fwd_t<float>(mode, x, y, rows, D, s);
  }
  gbh::set_error("gb_softmax_fwd: bad dtype %d", dtype);
  return gbh::E_BAD_ARG;
}

GB_EXPORT int gb_softmax_bwd(int mode, int dtype, const void* y, const void* dy, void* dx,
                             long long rows, int D, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (rows <= 0 || D <= 0) return gbh::E_OK;
  switch (dtype) {
    case DT_BF16: return softmax_bwd_t<__nv_bfloat16>(mode, y, dy, dx, rows, D, s);
    case DT_F16: return softmax_bwd_t<__half>(mode, y, dy, dx, rows, D, s);
    case DT_F32: return softmax_bwd_t<float>(mode, y, dy, dx, rows, D, s);
  }
  gbh::set_error("gb_softmax_bwd: bad dtype %d", dtype);
  return gbh::E_BAD_ARG;
}

// Cross-entropy forward.  out2 receives {loss, denominator}; reduction: 0 = mean,
// 1 = sum, 2 = none (loss_row holds the per-row values; out2 still filled with the sum).
GB_EXPORT int gb_ce_fwd(int dtype, const void* logits, const long long* targets,
                        const float* class_w, float class_w_sum, float* loss_row, float* lse,
                        float* w_row, float* out2, long long rows, int C, long long ignore_index,
                        int has_ignore, float label_smoothing, int reduction, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (rows <= 0 || C <= 0) return gbh::E_OK;
  if (!class_w) class_w_sum = (float)C;
  int rc;
  switch (dtype) {
    case DT_BF16: rc = ce_fwd_t<__nv_bfloat16>(logits, targets, class_w, loss_row, lse, w_row, rows, C, ignore_index, has_ignore, label_smoothing, class_w_sum, s); break;
    case DT_F16: rc = ce_fwd_t<__half>(logits, targets, class_w, loss_row, lse, w_row, rows, C, ignore_index, has_ignore, label_smoothing, class_w_sum, s); break;
    case DT_F32: rc = ce_fwd_t<float>(logits, targets, class_w, loss_row, lse, w_row, rows, C, ignore_index, has_ignore, label_smoothing, class_w_sum, s); break;
    default:
      gbh::set_error("gb_ce_fwd: bad dtype %d", dtype);
      return gbh::E_BAD_ARG;
  }
  if (rc) return rc;
  ce_reduce_kernel<<<1, 1024, 0, s>>>(loss_row, w_row, rows, reduction == 0, out2);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

// Loss and gradient at once (see ce_fused_vec_kernel): the logits are replaced by the gradient of the
// reduced loss (reduction 0 = mean over rows, 1 = sum); out2 = {loss, rows}.  Needs 16-bit logits,
// C a multiple of 8 and a 16-byte aligned buffer; returns E_BAD_ARG otherwise.
GB_EXPORT int gb_ce_fused(int dtype, void* logits, const long long* targets, float* loss_row, float* w_row,
                          float* out2, long long rows, int C, int reduction, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (rows <= 0 || C <= 0) return gbh::E_OK;
  if ((dtype != DT_BF16 && dtype != DT_F16) || (C & 7) || ((uintptr_t)logits & 15) || reduction > 1) {
    gbh::set_error("gb_ce_fused: 16-bit logits, a class count that is a multiple of 8, mean or sum");
    return gbh::E_BAD_ARG;
  }
  const float scale = reduction == 0 ? 1.f / (float)rows : 1.f;
  if (dtype == DT_BF16)
    ce_fused_vec_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, s>>>((__nv_bfloat16*)logits, targets, loss_row, w_row, C, scale, gbh::status_ptr());
  else
    ce_fused_vec_kernel<__half><<<(unsigned)rows, 256, 0, s>>>((__half*)logits, targets, loss_row, w_row, C, scale, gbh::status_ptr());
  GB_CUDA_OK(cudaGetLastError());
  ce_reduce_kernel<<<1, 1024, 0, s>>>(loss_row, w_row, rows, reduction == 0, out2);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

// x (n 16-bit elements, n a multiple of 8, 16-byte aligned) *= g[0], skipped on the device when g[0] == 1.
GB_EXPORT int gb_scale_unless_one(int dtype, void* x, long long n, const float* g, void* stream) {
  if (n <= 0) return gbh::E_OK;
  if ((dtype != DT_BF16 && dtype != DT_F16) || (n & 7) || ((uintptr_t)x & 15) || g == nullptr) {
    gbh::set_error("gb_scale_unless_one: 16-bit data, a multiple of 8 elements, 16-byte aligned");
    return gbh::E_BAD_ARG;
  }
  const long long nvec = n / 8;
  const int grid = (int)((nvec + 255) / 256 < 148 * 8 ? (nvec + 255) / 256 : 148 * 8);
  if (dtype == DT_BF16) scale_unless_one_kernel<__nv_bfloat16><<<grid, 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)x, nvec, g);
  else scale_unless_one_kernel<__half><<<grid, 256, 0, (cudaStream_t)stream>>>((__half*)x, nvec, g);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

// Cross-entropy backward.  g_scalar: upstream gradient of the reduced loss
// (device scalar) or null; g_row: per-row upstream gradient (reduction none)
// or null; denom: device scalar for the mean reduction or null.  dlogits may be
// the logits buffer itself.
GB_EXPORT int gb_ce_bwd(int dtype, const void* logits, const long long* targets,
                        const float* class_w, float class_w_sum, const float* lse,
                        const float* g_scalar, const float* g_row, const float* denom,
                        void* dlogits, long long rows, int C, long long ignore_index,
                        int has_ignore, float label_smoothing, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (rows <= 0 || C <= 0) return gbh::E_OK;
  if (!class_w) class_w_sum = (float)C;
  int blk = block_for(C);
#define GB_CE(T)                                                                                   \
  ce_bwd_kernel<T><<<(unsigned)rows, blk, 0, s>>>((const T*)logits, targets, class_w, lse, g_scalar, g_row, \
                                                  denom, (T*)dlogits, C, ignore_index, has_ignore,  \
                                                  label_smoothing, class_w_sum)
  switch (dtype) {
    case DT_BF16: GB_CE(__nv_bfloat16); break;
    case DT_F16: GB_CE(__half); break;
    case DT_F32: GB_CE(float); break;
    default:
      gbh::set_error("gb_ce_bwd: bad dtype %d", dtype);
      return gbh::E_BAD_ARG;
  }
#undef GB_CE
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}
