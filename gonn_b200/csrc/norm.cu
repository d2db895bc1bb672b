// LayerNorm / RMSNorm over the last dimension: one-pass forward that keeps the
// row in registers (statistics in fp32, variance from centred values), and a
// backward that produces dx and per-CTA partial sums of dgamma / dbeta, reduced
// by a second small kernel in a fixed order (deterministic).
//
// The reference composes these norms from ~10 elementwise / reduce tape nodes
// (nn/norm.go:50-78, 115-148); eps 1e-5 for LayerNorm, 1e-6 for RMSNorm, biased
// variance, RMSNorm = x / sqrt(mean(x^2) + eps) * w.
#include "common.cuh"

using namespace gb;

namespace {

template <typename T> struct IO;
template <> struct IO<__nv_bfloat16> {
  static constexpr int V = 8;
  using Raw = uint4;
  static __device__ __forceinline__ Raw ldraw(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }
  static __device__ __forceinline__ void unpack(const Raw& u, float* f) {
    float2 a;
    a = unpack_bf16(u.x); f[0] = a.x; f[1] = a.y;
    a = unpack_bf16(u.y); f[2] = a.x; f[3] = a.y;
    a = unpack_bf16(u.z); f[4] = a.x; f[5] = a.y;
    a = unpack_bf16(u.w); f[6] = a.x; f[7] = a.y;
  }
  static __device__ __forceinline__ void ld(const __nv_bfloat16* p, float* f) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    float2 a;
    a = unpack_bf16(u.x); f[0] = a.x; f[1] = a.y;
    a = unpack_bf16(u.y); f[2] = a.x; f[3] = a.y;
    a = unpack_bf16(u.z); f[4] = a.x; f[5] = a.y;
    a = unpack_bf16(u.w); f[6] = a.x; f[7] = a.y;
  }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, const float* f) {
    uint4 u;
    u.x = pack_bf16(f[0], f[1]); u.y = pack_bf16(f[2], f[3]);
    u.z = pack_bf16(f[4], f[5]); u.w = pack_bf16(f[6], f[7]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};
template <> struct IO<__half> {
  static constexpr int V = 8;
  using Raw = uint4;
  static __device__ __forceinline__ Raw ldraw(const __half* p) { return *reinterpret_cast<const uint4*>(p); }
  static __device__ __forceinline__ void unpack(const Raw& u, float* f) {
    float2 a;
    a = unpack_f16(u.x); f[0] = a.x; f[1] = a.y;
    a = unpack_f16(u.y); f[2] = a.x; f[3] = a.y;
    a = unpack_f16(u.z); f[4] = a.x; f[5] = a.y;
    a = unpack_f16(u.w); f[6] = a.x; f[7] = a.y;
  }
  static __device__ __forceinline__ void ld(const __half* p, float* f) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    float2 a;
    a = unpack_f16(u.x); f[0] = a.x; f[1] = a.y;
    a = unpack_f16(u.y); f[2] = a.x; f[3] = a.y;
    a = unpack_f16(u.z); f[4] = a.x; f[5] = a.y;
    a = unpack_f16(u.w); f[6] = a.x; f[7] = a.y;
  }
  static __device__ __forceinline__ void st(__half* p, const float* f) {
    uint4 u;
    u.x = pack_f16(f[0], f[1]); u.y = pack_f16(f[2], f[3]);
    u.z = pack_f16(f[4], f[5]); u.w = pack_f16(f[6], f[7]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};
template <> struct IO<float> {
  static constexpr int V = 4;
  using Raw = float4;
  static __device__ __forceinline__ Raw ldraw(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void unpack(const Raw& u, float* f) {
    f[0] = u.x; f[1] = u.y; f[2] = u.z; f[3] = u.w;
  }
  static __device__ __forceinline__ void ld(const float* p, float* f) {
    float4 u = *reinterpret_cast<const float4*>(p);
    f[0] = u.x; f[1] = u.y; f[2] = u.z; f[3] = u.w;
  }
  static __device__ __forceinline__ void st(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
};

// Reduction over the G threads that share a row (G = 32: a warp; G = 256: the
// whole CTA, through `red`).
template <int G>
__device__ __forceinline__ float group_sum(float v, float* red) {
  if (G == 32) return warp_sum(v);
  return block_sum(v, red);
}

// Forward.  A group of G threads owns one row; thread t of the group holds
// vectors t, t+G, ... (VPT of them) of the row in registers.
template <typename T, typename TW, int G, int VPT, bool RMS>
__global__ void __launch_bounds__(256)
norm_fwd_kernel(const T* __restrict__ x, const TW* __restrict__ w, const TW* __restrict__ b,
                T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                long long rows, int D, float eps) {
  constexpr int V = IO<T>::V;
  constexpr int NR = (G == 32) ? 2 : 4;  // rows in flight per group (more loads outstanding)
  __shared__ float red[32];
  const int gpb = 256 / G;
  const int g = threadIdx.x / G, t = threadIdx.x % G;
  const int nvec = D / V;
  // the thread's columns are the same for every row: keep weight and bias in registers
  float wr[VPT][V], br[VPT][V];
#pragma unroll
  for (int i = 0; i < VPT; i++) {
    const int vi = t + i * G;
#pragma unroll
    for (int j = 0; j < V; j++) {
      wr[i][j] = (w && vi < nvec) ? (float)w[vi * V + j] : 1.f;
      br[i][j] = (!RMS && b && vi < nvec) ? (float)b[vi * V + j] : 0.f;
    }
  }
  const long long stride = (long long)gridDim.x * gpb;
  for (long long row0 = (long long)blockIdx.x * gpb + g; row0 < rows; row0 += stride * NR) {
    float v[NR][VPT][V];
    float s[NR];
#pragma unroll
    for (int r = 0; r < NR; r++) {
      const long long row = row0 + r * stride;
      s[r] = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; i++) {
        const int vi = t + i * G;
        if (vi < nvec && row < rows) {
          IO<T>::ld(x + row * D + vi * V, v[r][i]);
        } else {
#pragma unroll
          for (int j = 0; j < V; j++) v[r][i][j] = 0.f;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < NR; r++) {
      const long long row = row0 + r * stride;
      if (row >= rows) continue;  // uniform across the group (a warp, or the whole CTA)
#pragma unroll
      for (int i = 0; i < VPT; i++)
#pragma unroll
        for (int j = 0; j < V; j++) s[r] += RMS ? v[r][i][j] * v[r][i][j] : v[r][i][j];
      const float sum = group_sum<G>(s[r], red);
      float mean = 0.f, rstd;
      if (RMS) {
        rstd = rsqrtf(sum / D + eps);
      } else {
        mean = sum / D;
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; i++) {
          const int vi = t + i * G;
          if (vi < nvec) {
#pragma unroll
            for (int j = 0; j < V; j++) { float d = v[r][i][j] - mean; q += d * d; }
          }
        }
        q = group_sum<G>(q, red);
        rstd = rsqrtf(q / D + eps);
      }
      if (t == 0) {
        if (mean_out) mean_out[row] = mean;
        rstd_out[row] = rstd;
      }
      T* yr = y + row * D;
#pragma unroll
      for (int i = 0; i < VPT; i++) {
        const int vi = t + i * G;
        if (vi < nvec) {
          float o[V];
#pragma unroll
          for (int j = 0; j < V; j++) o[j] = (v[r][i][j] - mean) * rstd * wr[i][j] + br[i][j];
          IO<T>::st(yr + vi * V, o);
        }
      }
    }
  }
}

// Backward.  dx per row; dgamma / dbeta accumulated per thread over the rows
// the group visits, then combined across the groups of the CTA in shared
// memory and written to part[blockIdx.x][2][D].
template <typename T, typename TW, int G, int VPT, bool RMS>
__global__ void __launch_bounds__(256, 2)
norm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy, const TW* __restrict__ w,
                const float* __restrict__ mean_in, const float* __restrict__ rstd_in,
                T* __restrict__ dx, float* __restrict__ part, long long rows, int D) {
  constexpr int V = IO<T>::V;
  extern __shared__ float sm[];  // [2][D] when G == 32
  __shared__ float red[32];
  const int gpb = 256 / G;
  const int g = threadIdx.x / G, t = threadIdx.x % G;
  const int nvec = D / V;
  float dg[VPT][V], db[VPT][V];
#pragma unroll
  for (int i = 0; i < VPT; i++)
#pragma unroll
    for (int j = 0; j < V; j++) { dg[i][j] = 0.f; db[i][j] = 0.f; }

  using Raw = typename IO<T>::Raw;
  const long long stride = (long long)gridDim.x * gpb;
  long long row = (long long)blockIdx.x * gpb + g;
  // Rows stay packed in registers (the arithmetic unpacks them twice) so that the next
  // row's loads can be in flight during this row's reductions without pushing the
  // register count past two CTAs per SM.
  Raw ax[VPT], ad[VPT], nx[VPT], nd[VPT];
  auto fetch = [&](long long r, Raw* px, Raw* pd) {
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int vi = t + i * G;
      if (vi < nvec && r < rows) {
        px[i] = IO<T>::ldraw(x + r * D + vi * V);
        pd[i] = IO<T>::ldraw(dy + r * D + vi * V);
      }
    }
  };
  constexpr bool PF = VPT * V <= 24;  // wider rows would spill with two rows resident
  if (PF) fetch(row, ax, ad);
  for (; row < rows; row += stride) {
    const float mean = RMS ? 0.f : mean_in[row];
    const float rstd = rstd_in[row];
    if (PF) fetch(row + stride, nx, nd);
    else fetch(row, ax, ad);
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int vi = t + i * G;
      if (vi < nvec) {
        float a[V], d[V];
        IO<T>::unpack(ax[i], a);
        IO<T>::unpack(ad[i], d);
#pragma unroll
        for (int j = 0; j < V; j++) {
          const float h = (a[j] - mean) * rstd;
          const float gw = w ? d[j] * (float)w[vi * V + j] : d[j];
          s1 += gw;
          s2 += gw * h;
          dg[i][j] += d[j] * h;
          db[i][j] += d[j];
        }
      }
    }
    if (!RMS) s1 = group_sum<G>(s1, red);
    s2 = group_sum<G>(s2, red);
    const float m1 = RMS ? 0.f : s1 / D, m2 = s2 / D;
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int vi = t + i * G;
      if (vi < nvec) {
        float a[V], d[V], o[V];
        IO<T>::unpack(ax[i], a);
        IO<T>::unpack(ad[i], d);
#pragma unroll
        for (int j = 0; j < V; j++) {
          const float h = (a[j] - mean) * rstd;
          const float gw = w ? d[j] * (float)w[vi * V + j] : d[j];
          o[j] = rstd * (gw - m1 - h * m2);
        }
        IO<T>::st(dx + row * D + vi * V, o);
      }
    }
    if (PF) {
#pragma unroll
      for (int i = 0; i < VPT; i++) { ax[i] = nx[i]; ad[i] = nd[i]; }
    }
  }
  if (part == nullptr) return;
  float* out = part + (long long)blockIdx.x * 2 * D;
  if (G == 32) {
    // combine the 8 warps of the CTA, one warp at a time
    for (int i = threadIdx.x; i < 2 * D; i += 256) sm[i] = 0.f;
    __syncthreads();
    for (int turn = 0; turn < gpb; turn++) {
      if (g == turn) {
#pragma unroll
        for (int i = 0; i < VPT; i++) {
          const int vi = t + i * G;
          if (vi < nvec) {
#pragma unroll
            for (int j = 0; j < V; j++) {
              sm[vi * V + j] += dg[i][j];
              sm[D + vi * V + j] += db[i][j];
            }
          }
        }
      }
      __syncthreads();
    }
    for (int i = threadIdx.x; i < 2 * D; i += 256) out[i] = sm[i];
  } else {
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int vi = t + i * G;
      if (vi < nvec) {
#pragma unroll
        for (int j = 0; j < V; j++) {
          out[vi * V + j] = dg[i][j];
          out[D + vi * V + j] = db[i][j];
        }
      }
    }
  }
}

// dgamma[c] = sum_p part[p][0][c], dbeta[c] = sum_p part[p][1][c]: CTA of 32 columns
// x 32 row lanes, fixed summation order.
template <typename TW>
__global__ void norm_param_reduce_kernel(const float* __restrict__ part, int P, int D,
                                         TW* __restrict__ dgamma, TW* __restrict__ dbeta) {
  __shared__ float sm[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (c < 2 * D)
    for (int p = threadIdx.y; p < P; p += 32) s += part[(long long)p * 2 * D + c];
  sm[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < 2 * D) {
#pragma unroll
    for (int k = 1; k < 32; k++) s += sm[k][threadIdx.x];
    if (c < D) {
      if (dgamma) dgamma[c] = (TW)s;
    } else if (dbeta) {
      dbeta[c - D] = (TW)s;
    }
  }
}

// Scalar fallback for D not a multiple of the vector width: one CTA per row.
template <typename T, typename TW, bool RMS>
__global__ void norm_fwd_generic(const T* __restrict__ x, const TW* __restrict__ w,
                                 const TW* __restrict__ b, T* __restrict__ y, float* mean_out,
                                 float* rstd_out, int D, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const T* xr = x + row * D;
  float s = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) { float v = (float)xr[i]; s += RMS ? v * v : v; }
  s = block_sum(s, red);
  float mean = 0.f, rstd;
  if (RMS) {
    rstd = rsqrtf(s / D + eps);
  } else {
    mean = s / D;
    float q = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) { float d = (float)xr[i] - mean; q += d * d; }
    q = block_sum(q, red);
    rstd = rsqrtf(q / D + eps);
  }
  if (threadIdx.x == 0) { if (mean_out) mean_out[row] = mean; rstd_out[row] = rstd; }
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float h = ((float)xr[i] - mean) * rstd;
    if (w) h *= (float)w[i];
    if (!RMS && b) h += (float)b[i];
    y[row * D + i] = (T)h;
  }
}

template <typename T, typename TW, bool RMS>
__global__ void norm_bwd_generic(const T* __restrict__ x, const T* __restrict__ dy,
                                 const TW* __restrict__ w, const float* mean_in,
                                 const float* rstd_in, T* __restrict__ dx, int D) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const float mean = RMS ? 0.f : mean_in[row], rstd = rstd_in[row];
  float s1 = 0.f, s2 = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float h = ((float)x[row * D + i] - mean) * rstd;
    float gw = (float)dy[row * D + i] * (w ? (float)w[i] : 1.f);
    s1 += gw; s2 += gw * h;
  }
  s1 = block_sum(s1, red);
  s2 = block_sum(s2, red);
  const float m1 = RMS ? 0.f : s1 / D, m2 = s2 / D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float h = ((float)x[row * D + i] - mean) * rstd;
    float gw = (float)dy[row * D + i] * (w ? (float)w[i] : 1.f);
    dx[row * D + i] = (T)(rstd * (gw - m1 - h * m2));
  }
}

// column sums of dy * xhat and dy for the generic path: thread per column
template <typename T, typename TW, bool RMS>
__global__ void norm_param_generic(const T* __restrict__ x, const T* __restrict__ dy,
                                   const float* mean_in, const float* rstd_in, long long rows, int D,
                                   TW* dgamma, TW* dbeta) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float g = 0.f, b = 0.f;
  for (long long r = 0; r < rows; r++) {
    float h = ((float)x[r * D + c] - (RMS ? 0.f : mean_in[r])) * rstd_in[r];
    float d = (float)dy[r * D + c];
    g += d * h; b += d;
  }
  if (dgamma) dgamma[c] = (TW)g;
  if (dbeta) dbeta[c] = (TW)b;
}

int pick_grid(long long rows, int gpb, int per_sm = 2) {
  long long need = (rows + gpb - 1) / gpb;
  long long cap = 148 * per_sm;
  return (int)(need < cap ? need : cap);
}

template <typename T, typename TW, bool RMS>
int norm_fwd_t(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd,
               long long rows, int D, float eps, cudaStream_t s) {
  constexpr int V = IO<T>::V;
  const bool aligned = (D % V == 0) && ((((uintptr_t)x | (uintptr_t)y) & 15) == 0);
  const int nvec = D / V;
#define GB_FWD(G, VPT)                                                                           \
  norm_fwd_kernel<T, TW, G, VPT, RMS><<<pick_grid(rows, 256 / G, 4), 256, 0, s>>>(               \
      (const T*)x, (const TW*)w, (const TW*)b, (T*)y, mean, rstd, rows, D, eps)
  if (aligned && nvec <= 32) GB_FWD(32, 1);
  else if (aligned && nvec <= 64) GB_FWD(32, 2);
  else if (aligned && nvec <= 96) GB_FWD(32, 3);
  else if (aligned && nvec <= 128) GB_FWD(32, 4);
  else if (aligned && nvec <= 256) GB_FWD(256, 1);
  else if (aligned && nvec <= 512) GB_FWD(256, 2);
  else if (aligned && nvec <= 1024) GB_FWD(256, 4);
  else
    norm_fwd_generic<T, TW, RMS><<<(unsigned)rows, 256, 0, s>>>((const T*)x, (const TW*)w,
                                                               (const TW*)b, (T*)y, mean, rstd, D, eps);
#undef GB_FWD
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

template <typename T, typename TW, bool RMS>
int norm_bwd_t(const void* x, const void* dy, const void* w, const float* mean, const float* rstd,
               void* dx, void* dgamma, void* dbeta, float* part, int part_rows, long long rows,
               int D, cudaStream_t s) {
  constexpr int V = IO<T>::V;
  const bool aligned = (D % V == 0) && ((((uintptr_t)x | (uintptr_t)dy | (uintptr_t)dx) & 15) == 0);
  const int nvec = D / V;
  const bool want_param = dgamma != nullptr || dbeta != nullptr;
  if (!aligned || nvec > 1024) {
    norm_bwd_generic<T, TW, RMS><<<(unsigned)rows, 256, 0, s>>>((const T*)x, (const T*)dy,
                                                               (const TW*)w, mean, rstd, (T*)dx, D);
    if (want_param)
      norm_param_generic<T, TW, RMS><<<(D + 127) / 128, 128, 0, s>>>(
          (const T*)x, (const T*)dy, mean, rstd, rows, D, (TW*)dgamma, (TW*)dbeta);
    GB_CUDA_OK(cudaGetLastError());
    return gbh::E_OK;
  }
  int grid = 0;
#define GB_BWD(G, VPT)                                                                           \
  {                                                                                              \
    grid = pick_grid(rows, 256 / G);                                                             \
    if (grid > part_rows) grid = part_rows;                                                      \
    size_t shm = (G == 32) ? 2 * (size_t)D * sizeof(float) : 0;                                  \
    norm_bwd_kernel<T, TW, G, VPT, RMS><<<grid, 256, shm, s>>>(                                  \
        (const T*)x, (const T*)dy, (const TW*)w, mean, rstd, (T*)dx, want_param ? part : nullptr, rows, D); \
  }
  if (want_param && (part == nullptr || part_rows < 1)) {
    gbh::set_error("norm backward: scratch for the parameter gradients is missing");
    return gbh::E_BAD_ARG;
  }
  if (!want_param) part_rows = 1 << 30;
  if (nvec <= 32) GB_BWD(32, 1)
  else if (nvec <= 64) GB_BWD(32, 2)
  else if (nvec <= 96) GB_BWD(32, 3)
  else if (nvec <= 128) GB_BWD(32, 4)
  else if (nvec <= 256) GB_BWD(256, 1)
  else if (nvec <= 512) GB_BWD(256, 2)
  else GB_BWD(256, 4)
#undef GB_BWD
  GB_CUDA_OK(cudaGetLastError());
  if (want_param) {
    norm_param_reduce_kernel<TW><<<(2 * D + 31) / 32, dim3(32, 32), 0, s>>>(part, grid, D, (TW*)dgamma,
                                                                           (TW*)dbeta);
    GB_CUDA_OK(cudaGetLastError());
  }
  return gbh::E_OK;
}

}  // namespace

enum { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2 };

// Maximum number of partial rows the backward may use; scratch must hold
// gb_norm_bwd_scratch_rows() * 2 * D floats.
GB_EXPORT int gb_norm_bwd_scratch_rows() { return 148 * 2; }

// kind: 0 = LayerNorm, 1 = RMSNorm.  dtype of x / y; wdtype of weight / bias
// (the same as dtype, or fp32).  mean may be null for RMSNorm.
GB_EXPORT int gb_norm_fwd(int kind, int dtype, int wdtype, const void* x, const void* w,
                          const void* b, void* y, float* mean, float* rstd, long long rows, int D,
                          float eps, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (rows <= 0 || D <= 0) return gbh::E_OK;
#define GB_N(DTI, T, WDI, TW)                                                              \
  if (dtype == DTI && wdtype == WDI)                                                       \
    return kind ? norm_fwd_t<T, TW, true>(x, w, b, y, mean, rstd, rows, D, eps, s)         \
                : norm_fwd_t<T, TW, false>(x, w, b, y, mean, rstd, rows, D, eps, s);
  GB_N(DT_BF16, __nv_bfloat16, DT_BF16, __nv_bfloat16)
  GB_N(DT_BF16, __nv_bfloat16, DT_F32, float)
  GB_N(DT_F16, __half, DT_F16, __half)
  GB_N(DT_F16, __half, DT_F32, float)
  GB_N(DT_F32, float, DT_F32, float)
#undef GB_N
  gbh::set_error("gb_norm_fwd: unsupported dtype pair %d/%d", dtype, wdtype);
  return gbh::E_BAD_ARG;
}

GB_EXPORT int gb_norm_bwd(int kind, int dtype, int wdtype, const void* x, const void* dy,
                          const void* w, const float* mean, const float* rstd, void* dx,
                          void* dgamma, void* dbeta, float* scratch, int scratch_rows,
                          long long rows, int D, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (rows <= 0 || D <= 0) return gbh::E_OK;
#define GB_N(DTI, T, WDI, TW)                                                                        \
  if (dtype == DTI && wdtype == WDI)                                                                 \
    return kind ? norm_bwd_t<T, TW, true>(x, dy, w, mean, rstd, dx, dgamma, dbeta, scratch,          \
                                          scratch_rows, rows, D, s)                                  \
                : norm_bwd_t<T, TW, false>(x, dy, w, mean, rstd, dx, dgamma, dbeta, scratch,         \
                                           scratch_rows, rows, D, s);
  GB_N(DT_BF16, __nv_bfloat16, DT_BF16, __nv_bfloat16)
  GB_N(DT_BF16, __nv_bfloat16, DT_F32, float)
  GB_N(DT_F16, __half, DT_F16, __half)
  GB_N(DT_F16, __half, DT_F32, float)
  GB_N(DT_F32, float, DT_F32, float)
#undef GB_N
  gbh::set_error("gb_norm_bwd: unsupported dtype pair %d/%d", dtype, wdtype);
  return gbh::E_BAD_ARG;
}

// ---------------------------------------------------------------------------
// LayerNorm / RMSNorm backward without any allocation (see norm_noalloc.h)
// ---------------------------------------------------------------------------
// The partial dgamma / dbeta sums of the backward kernel normally live in a
// buffer the caller allocates.  This variant keeps them in a fixed array inside
// the library image instead.  Every GPU that loads the library holds the array
// (kNoAllocRows * 2 * kNoAllocMaxD floats, about 4.6 MiB) until the process exits.
namespace {
constexpr int kNoAllocRows = 148;    // partial rows: at most one CTA per SM
constexpr int kNoAllocMaxD = 4096;   // widest row this entry point accepts
constexpr int kNoAllocDevices = 16;
static __device__ __align__(256) float g_noalloc_scratch[(size_t)kNoAllocRows * 2 * kNoAllocMaxD];
// Device address of the array per device.  In host code the array's name only stands in
// for the symbol; the address a kernel can use comes from cudaGetSymbolAddress.
float* g_noalloc_ptr[kNoAllocDevices] = {nullptr};
}  // namespace

GB_EXPORT int gb_norm_bwd_noalloc_max_dim() { return kNoAllocMaxD; }

GB_EXPORT int gb_norm_bwd_noalloc(int kind, int dtype, int wdtype, const void* x, const void* dy,
                                  const void* w, const float* mean, const float* rstd, void* dx,
                                  void* dgamma, void* dbeta, long long rows, int D, void* stream) {
  if (D > kNoAllocMaxD) {
    gbh::set_error("gb_norm_bwd_noalloc: row width %d exceeds the built-in scratch (max %d)", D,
                   kNoAllocMaxD);
    return gbh::E_TOO_LARGE;
  }
  int dev = 0;
  GB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kNoAllocDevices) {
    gbh::set_error("gb_norm_bwd_noalloc: device index %d out of range", dev);
    return gbh::E_BAD_ARG;
  }
  if (g_noalloc_ptr[dev] == nullptr) {
    // one-time set-up for this device (it is the current device here)
    float* p = nullptr;
    GB_CUDA_OK(cudaGetSymbolAddress((void**)&p, g_noalloc_scratch));
    g_noalloc_ptr[dev] = p;
  }
  // The kernels write every partial row they later read, so nothing needs clearing.
  return gb_norm_bwd(kind, dtype, wdtype, x, dy, w, mean, rstd, dx, dgamma, dbeta, g_noalloc_ptr[dev],
                     kNoAllocRows, rows, D, stream);
}
