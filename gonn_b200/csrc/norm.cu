// LayerNorm / RMSNorm over the last dimension: one-pass forward that keeps the
// row in registers (statistics in fp32, variance from centred values), and a
// backward that produces dx and per-CTA partial sums of dgamma / dbeta, reduced
// by a second small kernel in a fixed order (deterministic).
//
// The reference composes these norms from ~10 elementwise / reduce tape nodes
// (nn/norm.go:50-78, 115-148); eps 1e-5 for LayerNorm, 1e-6 for RMSNorm, biased
// variance, RMSNorm = x / sqrt(mean(x^2) + eps) * w.
#include "bounds.cuh"

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
  if (!GB_IN_EXTENT(blockIdx.x, 0, 401)) return;   // more CTAs than partial rows in the scratch
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

// dgamma[c] = sum_p part[p][0][c], dbeta[c] = sum_p part[p][1][c] (and dsum[c] from
// part[p][2][c] when NP == 3): CTA of 32 columns x 32 row lanes, fixed summation order.
template <typename TW, typename TS>
__global__ void norm_param_reduce_kernel(const float* __restrict__ part, int P, int D, int NP,
                                         TW* __restrict__ dgamma, TW* __restrict__ dbeta,
                                         TS* __restrict__ dsum, int dsum_accumulate) {
  __shared__ float sm[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (c < NP * D)
    for (int p = threadIdx.y; p < P; p += 32) s += part[(long long)p * NP * D + c];
  sm[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < NP * D) {
#pragma unroll
    for (int k = 1; k < 32; k++) s += sm[k][threadIdx.x];
    if (c < D) {
      if (dgamma) dgamma[c] = (TW)s;
    } else if (c < 2 * D) {
      if (dbeta) dbeta[c - D] = (TW)s;
    } else if (dsum) {
      dsum[c - 2 * D] = dsum_accumulate ? (TS)((float)dsum[c - 2 * D] + s) : (TS)s;
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

// ---------------------------------------------------------------------------
// Pipelined kernels (the fast path): a producer warp streams tiles of whole rows
// into a ring of shared-memory stages with bulk asynchronous copies (rows of a
// contiguous matrix are one contiguous byte range, so no tensor map is needed),
// 256 consumer threads take rows out of the ring.  Memory-level parallelism is
// set by the ring (stages x tile bytes in flight per CTA), not by the number of
// resident warps.  A group of G consumer threads owns one row (G = 32 .. 256 by
// row width); thread t of the group keeps vectors t, t+G, ... packed in registers.
// ---------------------------------------------------------------------------
constexpr int kPipeConsumers = 256;
constexpr int kPipeThreads = kPipeConsumers + 32;
constexpr int kPipeMaxStages = 8;
constexpr int kPipeHeader = 1024;  // barriers, abort flag, reduction slots

__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"((uint64_t)src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

struct PipeSmem {
  uint64_t full[kPipeMaxStages];
  uint64_t empty[kPipeMaxStages];
  int abort_flag;
  int pad[3];
  float first[4];
  float2 red[2][4][8];  // [flip][group][warp in group]; groups of one warp need no slot
};
static_assert(sizeof(PipeSmem) <= kPipeHeader, "header too small");

// Sum of a pair over the G threads of a group, same value in every thread, fixed order.
template <int G>
__device__ __forceinline__ float2 group_sum2(float2 v, PipeSmem* ps, int g, int& flip) {
  v.x = warp_sum(v.x);
  v.y = warp_sum(v.y);
  if (G == 32) return v;
  constexpr int NW = G / 32;
  const int wig = (threadIdx.x % G) >> 5;
  float2* slot = ps->red[flip][g];
  if ((threadIdx.x & 31) == 0) slot[wig] = v;
  named_bar_sync(1 + g, G);
  float2 r = make_float2(0.f, 0.f);
#pragma unroll
  for (int j = 0; j < NW; j++) { r.x += slot[j].x; r.y += slot[j].y; }
  flip ^= 1;  // the other slot set next time: no second barrier needed before reuse
  return r;
}

// V consecutive weights starting at vector vi, widened to fp32 (vector loads from shared memory)
// The first element of the row (held by thread 0 of the group) for every thread of a group
// wider than a warp.  Uses its own slot so that it does not disturb group_sum2's double buffer.
template <int G>
__device__ __forceinline__ float ps_first_of_row(float k_lane0, PipeSmem* ps, int g) {
  if ((threadIdx.x % G) == 0) ps->first[g] = k_lane0;
  named_bar_sync(1 + g, G);
  const float k = ps->first[g];
  named_bar_sync(1 + g, G);
  return k;
}

template <typename TW, int V>
__device__ __forceinline__ void load_wvec(const TW* sw, int vi, float* f) {
  if constexpr (sizeof(TW) == 2) {
    static_assert(V == 8, "16-bit weights come with 16-bit rows");
    IO<TW>::unpack(*reinterpret_cast<const uint4*>(sw + vi * 8), f);
  } else {
#pragma unroll
    for (int j = 0; j < V; j += 4) {
      const float4 u = *reinterpret_cast<const float4*>(sw + vi * V + j);
      f[j] = u.x; f[j + 1] = u.y; f[j + 2] = u.z; f[j + 3] = u.w;
    }
  }
}

// Producer loop shared by forward and backward: `nsrc` source matrices per stage.
template <int NSRC>
__device__ __forceinline__ void pipe_produce(PipeSmem* ps, unsigned char* stages, size_t stage_bytes,
                                             size_t src_bytes_per_tile, const unsigned char* s0,
                                             const unsigned char* s1, const unsigned char* s2, long long rows, int R,
                                             size_t row_bytes, int S, int* status) {
  const long long ntiles = (rows + R - 1) / R;
  int it = 0;
  for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x, it++) {
    const int s = it % S;
    const uint32_t ph = (uint32_t)(it / S) & 1u;
    if (!mbar_wait(&ps->empty[s], ph ^ 1u, &ps->abort_flag, status, ST_NORM_TIMEOUT, 10 + s)) return;
    const long long r0 = tile * R;
    const long long nr = (rows - r0 < R) ? (rows - r0) : R;
    const uint32_t bytes = (uint32_t)(nr * row_bytes);
    mbar_expect_tx(&ps->full[s], bytes * NSRC);
    unsigned char* dst = stages + (size_t)s * stage_bytes;
    bulk_load(dst, s0 + (size_t)r0 * row_bytes, bytes, &ps->full[s]);
    if (NSRC >= 2) bulk_load(dst + src_bytes_per_tile, s1 + (size_t)r0 * row_bytes, bytes, &ps->full[s]);
    if (NSRC >= 3) bulk_load(dst + 2 * src_bytes_per_tile, s2 + (size_t)r0 * row_bytes, bytes, &ps->full[s]);
  }
}

// Packed fp32 pairs: one instruction handles two lanes of arithmetic (add / mul / fma on
// float2 operands), which halves the issue slots of these kernels; the measured limiter of a
// first version with scalar arithmetic was instruction issue, not memory.
__device__ __forceinline__ float2 f2(float a) { return make_float2(a, a); }
template <typename T> struct Pairs;   // a 16-byte vector as V/2 float2 pairs
template <> struct Pairs<__nv_bfloat16> {
  static constexpr int NP2 = 4;
  static __device__ __forceinline__ void unpack(const uint4& u, float2* f) {
    f[0] = unpack_bf16(u.x); f[1] = unpack_bf16(u.y); f[2] = unpack_bf16(u.z); f[3] = unpack_bf16(u.w);
  }
  static __device__ __forceinline__ uint4 pack(const float2* f) {
    uint4 u;
    u.x = pack_bf16(f[0].x, f[0].y); u.y = pack_bf16(f[1].x, f[1].y);
    u.z = pack_bf16(f[2].x, f[2].y); u.w = pack_bf16(f[3].x, f[3].y);
    return u;
  }
};
template <> struct Pairs<__half> {
  static constexpr int NP2 = 4;
  static __device__ __forceinline__ void unpack(const uint4& u, float2* f) {
    f[0] = unpack_f16(u.x); f[1] = unpack_f16(u.y); f[2] = unpack_f16(u.z); f[3] = unpack_f16(u.w);
  }
  static __device__ __forceinline__ uint4 pack(const float2* f) {
    uint4 u;
    u.x = pack_f16(f[0].x, f[0].y); u.y = pack_f16(f[1].x, f[1].y);
    u.z = pack_f16(f[2].x, f[2].y); u.w = pack_f16(f[3].x, f[3].y);
    return u;
  }
};
template <> struct Pairs<float> {
  static constexpr int NP2 = 2;
  static __device__ __forceinline__ void unpack(const float4& u, float2* f) {
    f[0] = make_float2(u.x, u.y); f[1] = make_float2(u.z, u.w);
  }
  static __device__ __forceinline__ float4 pack(const float2* f) {
    return make_float4(f[0].x, f[0].y, f[1].x, f[1].y);
  }
};
// NP2 pairs of fp32 constants (weights widened once per CTA) from shared memory
template <int NP2>
__device__ __forceinline__ void load_pairs(const float* s, int vi, float2* f) {
#pragma unroll
  for (int j = 0; j < NP2; j += 2) {
    const float4 u = *reinterpret_cast<const float4*>(s + vi * NP2 * 2 + j * 2);
    f[j] = make_float2(u.x, u.y);
    f[j + 1] = make_float2(u.z, u.w);
  }
}

template <typename T, typename TW, int G, int VPT, bool RMS>
__global__ void __launch_bounds__(kPipeThreads, 3)
norm_fwd_pipe_kernel(const T* __restrict__ x, const TW* __restrict__ w, const TW* __restrict__ b,
                     T* __restrict__ y, float* __restrict__ mean_out, float* __restrict__ rstd_out,
                     long long rows, int D, float eps, int KR, int S, int* status) {
  constexpr int V = IO<T>::V;
  constexpr int NP2 = Pairs<T>::NP2;
  constexpr int NG = kPipeConsumers / G;
  using Raw = typename IO<T>::Raw;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  PipeSmem* ps = reinterpret_cast<PipeSmem*>(smem_raw);
  const int R = NG * KR;
  const size_t row_bytes = (size_t)D * sizeof(T);
  const size_t stage_bytes = (size_t)R * row_bytes;
  unsigned char* stages = smem_raw + kPipeHeader;
  float* sw = reinterpret_cast<float*>(stages + (size_t)S * stage_bytes);  // weights, widened
  float* sb = sw + D;
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) { mbar_init(&ps->full[s], 1); mbar_init(&ps->empty[s], kPipeConsumers / 32); }
    ps->abort_flag = 0;
    mbar_fence_init();
  }
  for (int i = threadIdx.x; i < D; i += kPipeThreads) {
    sw[i] = w ? (float)w[i] : 1.f;
    sb[i] = (!RMS && b) ? (float)b[i] : 0.f;
  }
  __syncthreads();
  if (threadIdx.x >= kPipeConsumers) {
    if (threadIdx.x == kPipeConsumers)
      pipe_produce<1>(ps, stages, stage_bytes, 0, (const unsigned char*)x, nullptr, nullptr, rows, R, row_bytes, S,
                      status);
    return;
  }
  const int g = threadIdx.x / G, t = threadIdx.x % G;
  const int nvec = D / V;
  const float invD = 1.f / (float)D;
  const long long ntiles = (rows + R - 1) / R;
  int flip = 0, it = 0;
  for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x, it++) {
    const int s = it % S;
    const uint32_t ph = (uint32_t)(it / S) & 1u;
    if (!mbar_wait(&ps->full[s], ph, &ps->abort_flag, status, ST_NORM_TIMEOUT, s)) return;
    const unsigned char* st = stages + (size_t)s * stage_bytes;
    for (int kk = 0; kk < KR; kk++) {
      const int r = kk * NG + g;
      const long long row = tile * R + r;
      const bool live = row < rows;  // uniform over the group
      float2 f[VPT][NP2];
      if (live) {
#pragma unroll
        for (int i = 0; i < VPT; i++) {
          const int vi = t + i * G;
          if (vi < nvec) {
            Pairs<T>::unpack(*reinterpret_cast<const Raw*>(st + (size_t)r * row_bytes + (size_t)vi * sizeof(Raw)), f[i]);
          } else {
#pragma unroll
            for (int j = 0; j < NP2; j++) f[i][j] = f2(0.f);
          }
        }
      }
      if (kk == KR - 1) {  // every row of the stage is in registers: hand the stage back
        __syncwarp();
        if ((threadIdx.x & 31) == 0) mbar_arrive(&ps->empty[s]);
      }
      if (!live) continue;
      float mean = 0.f, rstd, shiftv = 0.f;
      if (RMS) {
        float2 q = f2(0.f);
#pragma unroll
        for (int i = 0; i < VPT; i++)
#pragma unroll
          for (int j = 0; j < NP2; j++) q = __ffma2_rn(f[i][j], f[i][j], q);
        float2 tot = group_sum2<G>(make_float2(q.x + q.y, 0.f), ps, g, flip);
        rstd = rsqrtf(tot.x * invD + eps);
      } else {
        // One pass, one reduction: sums of (x - K) and (x - K)^2 with K = the row's first
        // element, so that the variance E[(x-K)^2] - E[x-K]^2 does not cancel when the mean
        // is large against the spread (K is within the spread of the row).
        const float K = __shfl_sync(0xffffffffu, f[0][0].x, 0);   // lane 0 of every warp holds vector t = 32 w, ...
        const float K0 = (G == 32) ? K : ps_first_of_row<G>(K, ps, g);
        const float2 nk = f2(-K0);
        float2 a = f2(0.f), q = f2(0.f);
#pragma unroll
        for (int i = 0; i < VPT; i++) {
          if (t + i * G < nvec) {
#pragma unroll
            for (int j = 0; j < NP2; j++) {
              f[i][j] = __fadd2_rn(f[i][j], nk);
              a = __fadd2_rn(a, f[i][j]);
              q = __ffma2_rn(f[i][j], f[i][j], q);
            }
          }
        }
        const float2 tot = group_sum2<G>(make_float2(a.x + a.y, q.x + q.y), ps, g, flip);
        const float m = tot.x * invD;            // mean of the shifted row
        mean = K0 + m;
        rstd = rsqrtf(fmaxf(tot.y * invD - m * m, 0.f) + eps);
        shiftv = -m * rstd;
      }
      if (t == 0) {
        if (mean_out) mean_out[row] = mean;
        rstd_out[row] = rstd;
      }
      T* yr = y + row * D;
      const float2 rs = f2(rstd), sv = f2(shiftv);
#pragma unroll
      for (int i = 0; i < VPT; i++) {
        const int vi = t + i * G;
        if (vi < nvec) {
          float2 wv[NP2], bv[NP2], o[NP2];
          load_pairs<NP2>(sw, vi, wv);
          load_pairs<NP2>(sb, vi, bv);
#pragma unroll
          for (int j = 0; j < NP2; j++) o[j] = __ffma2_rn(__ffma2_rn(f[i][j], rs, sv), wv[j], bv[j]);
          *reinterpret_cast<Raw*>(yr + vi * V) = Pairs<T>::pack(o);
        }
      }
    }
  }
}

// Backward: dx per row; dgamma / dbeta accumulate per thread over the rows its group
// visits, are combined over the groups of the CTA through shared memory in group order and
// written to part[blockIdx.x][NP][D]; norm_param_reduce_kernel adds the CTAs in index order.
// RES: a third stream `dres` (the gradient that bypassed the norm through a residual
// connection) is added to dx, and its column sums go to part[..][2][D]: they are the bias
// gradient of the linear layer whose output was added to the residual stream after this norm.
template <typename T, typename TW, int G, int VPT, bool RMS, bool RES>
__global__ void __launch_bounds__(kPipeThreads, 2)
norm_bwd_pipe_kernel(const T* __restrict__ x, const T* __restrict__ dy, const T* __restrict__ dres,
                     const TW* __restrict__ w, const float* __restrict__ mean_in,
                     const float* __restrict__ rstd_in, T* __restrict__ dx, float* __restrict__ part,
                     long long rows, int D, int KR, int S, int* status) {
  constexpr int NP = RES ? 3 : 2;  // partial rows per CTA: dgamma, dbeta (, column sums of dres)
  constexpr int V = IO<T>::V;
  constexpr int NP2 = Pairs<T>::NP2;
  constexpr int NG = kPipeConsumers / G;
  using Raw = typename IO<T>::Raw;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  PipeSmem* ps = reinterpret_cast<PipeSmem*>(smem_raw);
  const int R = NG * KR;
  const size_t row_bytes = (size_t)D * sizeof(T);
  const size_t half_bytes = (size_t)R * row_bytes;
  const size_t stage_bytes = NP * half_bytes;
  unsigned char* stages = smem_raw + kPipeHeader;
  float* sw = reinterpret_cast<float*>(stages + (size_t)S * stage_bytes);
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) { mbar_init(&ps->full[s], 1); mbar_init(&ps->empty[s], kPipeConsumers / 32); }
    ps->abort_flag = 0;
    mbar_fence_init();
  }
  for (int i = threadIdx.x; i < D; i += kPipeThreads) sw[i] = w ? (float)w[i] : 1.f;
  __syncthreads();
  const bool producer = threadIdx.x >= kPipeConsumers;
  if (threadIdx.x == kPipeConsumers)
    pipe_produce<NP>(ps, stages, stage_bytes, half_bytes, (const unsigned char*)x, (const unsigned char*)dy,
                     (const unsigned char*)dres, rows, R, row_bytes, S, status);
  const int g = threadIdx.x / G, t = threadIdx.x % G;
  const int nvec = D / V;
  const float invD = 1.f / (float)D;
  float2 dg[VPT][NP2], db[VPT][NP2], ds[RES ? VPT : 1][NP2];
#pragma unroll
  for (int i = 0; i < VPT; i++)
#pragma unroll
    for (int j = 0; j < NP2; j++) { dg[i][j] = f2(0.f); db[i][j] = f2(0.f); if (RES) ds[i][j] = f2(0.f); }
  if (!producer) {
    const long long ntiles = (rows + R - 1) / R;
    int flip = 0, it = 0;
    for (long long tile = blockIdx.x; tile < ntiles; tile += gridDim.x, it++) {
      const int s = it % S;
      const uint32_t ph = (uint32_t)(it / S) & 1u;
      // the row statistics of this tile's first row are fetched before the wait
      const long long row_first = tile * R + g;
      float mean_n = 0.f, rstd_n = 0.f;
      if (row_first < rows) { mean_n = RMS ? 0.f : mean_in[row_first]; rstd_n = rstd_in[row_first]; }
      if (!mbar_wait(&ps->full[s], ph, &ps->abort_flag, status, ST_NORM_TIMEOUT, 20 + s)) break;
      const unsigned char* st = stages + (size_t)s * stage_bytes;
      for (int kk = 0; kk < KR; kk++) {
        const int r = kk * NG + g;
        const long long row = tile * R + r;
        const bool live = row < rows;
        Raw xr[VPT], dr[VPT], rr[RES ? VPT : 1];
        if (live) {
#pragma unroll
          for (int i = 0; i < VPT; i++) {
            const int vi = t + i * G;
            if (vi < nvec) {
              const unsigned char* src = st + (size_t)r * row_bytes + (size_t)vi * sizeof(Raw);
              xr[i] = *reinterpret_cast<const Raw*>(src);
              dr[i] = *reinterpret_cast<const Raw*>(src + half_bytes);
              if (RES) rr[i] = *reinterpret_cast<const Raw*>(src + 2 * half_bytes);
            }
          }
        }
        if (kk == KR - 1) {
          __syncwarp();
          if ((threadIdx.x & 31) == 0) mbar_arrive(&ps->empty[s]);
        }
        const float mean = mean_n, rstd = rstd_n;
        const long long row_next = row + NG;
        if (kk + 1 < KR && row_next < rows) { mean_n = RMS ? 0.f : mean_in[row_next]; rstd_n = rstd_in[row_next]; }
        if (!live) continue;
        const float2 rs = f2(rstd), sh = f2(-mean * rstd);
        // h = normalised input, gw = dy * weight: both stay in registers for the second pass
        float2 h[VPT][NP2], gw[VPT][NP2];
        float2 s1 = f2(0.f), s2 = f2(0.f);
#pragma unroll
        for (int i = 0; i < VPT; i++) {
          const int vi = t + i * G;
          if (vi < nvec) {
            float2 d[NP2], wv[NP2];
            Pairs<T>::unpack(xr[i], h[i]);
            Pairs<T>::unpack(dr[i], d);
            load_pairs<NP2>(sw, vi, wv);
#pragma unroll
            for (int j = 0; j < NP2; j++) {
              h[i][j] = __ffma2_rn(h[i][j], rs, sh);
              gw[i][j] = __fmul2_rn(d[j], wv[j]);
              s1 = __fadd2_rn(s1, gw[i][j]);
              s2 = __ffma2_rn(gw[i][j], h[i][j], s2);
              dg[i][j] = __ffma2_rn(d[j], h[i][j], dg[i][j]);
              db[i][j] = __fadd2_rn(db[i][j], d[j]);
            }
          }
        }
        const float2 tot = group_sum2<G>(make_float2(s1.x + s1.y, s2.x + s2.y), ps, g, flip);
        const float m1 = RMS ? 0.f : tot.x * invD, m2 = tot.y * invD;
        // dx = rstd * (gw - m1 - h * m2) = gw * rstd + (h * (-rstd m2) + (-rstd m1))
        const float2 c2 = f2(-rstd * m2), c1 = f2(-rstd * m1);
#pragma unroll
        for (int i = 0; i < VPT; i++) {
          const int vi = t + i * G;
          if (vi < nvec) {
            float2 o[NP2];
#pragma unroll
            for (int j = 0; j < NP2; j++) o[j] = __ffma2_rn(gw[i][j], rs, __ffma2_rn(h[i][j], c2, c1));
            if (RES) {
              float2 e[NP2];
              Pairs<T>::unpack(rr[i], e);
#pragma unroll
              for (int j = 0; j < NP2; j++) { o[j] = __fadd2_rn(o[j], e[j]); ds[i][j] = __fadd2_rn(ds[i][j], e[j]); }
            }
            *reinterpret_cast<Raw*>(dx + row * D + vi * V) = Pairs<T>::pack(o);
          }
        }
      }
    }
  }
  if (part == nullptr) return;
  // every tile this CTA was given has been consumed (or the CTA is unwinding after a
  // time-out, in which case the status word already says so): the ring is free for reuse
  __syncthreads();
  float* comb = reinterpret_cast<float*>(stages);  // [NG][NP][D]
  if (!producer) {
#pragma unroll
    for (int i = 0; i < VPT; i++) {
      const int vi = t + i * G;
      if (vi < nvec) {
#pragma unroll
        for (int j = 0; j < NP2; j++) {
          const int c = vi * V + 2 * j;
          *reinterpret_cast<float2*>(comb + ((size_t)g * NP + 0) * D + c) = dg[i][j];
          *reinterpret_cast<float2*>(comb + ((size_t)g * NP + 1) * D + c) = db[i][j];
          if (RES) *reinterpret_cast<float2*>(comb + ((size_t)g * NP + 2) * D + c) = ds[i][j];
        }
      }
    }
  }
  __syncthreads();
  if (!GB_IN_EXTENT(blockIdx.x, 0, 402)) return;   // more CTAs than partial rows in the scratch
  float* out = part + (long long)blockIdx.x * NP * D;
  for (int c = threadIdx.x; c < NP * D; c += kPipeThreads) {
    float sacc = 0.f;
#pragma unroll
    for (int gg = 0; gg < NG; gg++) sacc += comb[(size_t)gg * NP * D + c];
    out[c] = sacc;
  }
}

// Geometry of the pipelined kernels for a row of `row_bytes`: rows per group per tile
// (tiles of about 12 KB per source), ring depth within `budget` bytes of shared memory.
struct PipePlan { int KR, S; size_t smem; bool ok; };
inline PipePlan pipe_plan(size_t row_bytes, int NG, int nsrc, size_t extra_bytes, size_t comb_bytes,
                          size_t limit = 110 * 1024, size_t target = 96 * 1024) {
  PipePlan p;
  const size_t tile = (size_t)NG * row_bytes;
  p.KR = 1;
  while ((size_t)(p.KR * 2) * tile <= 12288) p.KR *= 2;
  const size_t stage = (size_t)p.KR * tile * nsrc;
  // limit: shared memory one CTA may take (110 KB: two CTAs per SM; 72 KB: three); target: ring size
  const size_t avail = limit > kPipeHeader + extra_bytes ? limit - kPipeHeader - extra_bytes : 0;
  int S = (int)(avail / stage);
  if (S > kPipeMaxStages) S = kPipeMaxStages;
  while (S > 2 && (size_t)S * stage > target && (size_t)(S - 1) * stage >= comb_bytes) S--;
  p.S = S;
  p.smem = kPipeHeader + (size_t)S * stage + extra_bytes;
  // the combine buffer of the backward reuses the ring once it has drained
  p.ok = S >= 2 && (size_t)S * stage >= comb_bytes && p.smem <= limit;
  return p;
}

// (threads per row, vectors per thread) by row width in 16-byte vectors.  The backward keeps
// 16 fp32 accumulators per vector in registers, so it spreads a row over more threads.
#define GB_PIPE_DISPATCH(X)      \
  if (nvec <= 32) X(32, 1)       \
  else if (nvec <= 64) X(32, 2)  \
  else if (nvec <= 96) X(32, 3)  \
  else if (nvec <= 128) X(64, 2) \
  else if (nvec <= 192) X(64, 3) \
  else if (nvec <= 256) X(128, 2)\
  else if (nvec <= 384) X(128, 3)\
  else if (nvec <= 512) X(256, 2)\
  else if (nvec <= 768) X(256, 3)\
  else X(256, 4)
#define GB_PIPE_DISPATCH_BWD(X)  \
  if (nvec <= 32) X(32, 1)       \
  else if (nvec <= 64) X(32, 2)  \
  else if (nvec <= 128) X(64, 2) \
  else if (nvec <= 256) X(128, 2)\
  else if (nvec <= 512) X(256, 2)\
  else if (nvec <= 768) X(256, 3)\
  else X(256, 4)

#define GB_PIPE_DISPATCH_RES(X)  \
  if (nvec <= 32) X(32, 1)       \
  else if (nvec <= 64) X(64, 1)  \
  else if (nvec <= 128) X(128, 1)\
  else if (nvec <= 256) X(256, 1)\
  else if (nvec <= 512) X(256, 2)\
  else if (nvec <= 768) X(256, 3)\
  else X(256, 4)

bool g_norm_pipe = true;  // gb_norm_tune: 0 selects the register-resident kernels without the ring

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
  if (aligned && nvec <= 1024 && g_norm_pipe) {
    int rc = 1;
#define GB_FWDP(G, VPT)                                                                                  \
    {                                                                                                    \
      PipePlan pl = pipe_plan((size_t)D * sizeof(T), kPipeConsumers / G, 1, 2 * (size_t)D * sizeof(float), 0, \
                              72 * 1024, 56 * 1024); \
      if (pl.ok) {                                                                                       \
        auto kern = norm_fwd_pipe_kernel<T, TW, G, VPT, RMS>;                                            \
        static bool attr_set = false;                                                                    \
        if (!attr_set) {                                                                                 \
          GB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024)); \
          attr_set = true;                                                                               \
        }                                                                                                \
        const long long ntiles = (rows + (kPipeConsumers / G) * pl.KR - 1) / ((kPipeConsumers / G) * pl.KR); \
        const int grid = (int)(ntiles < 444 ? ntiles : 444);                                             \
        kern<<<grid, kPipeThreads, pl.smem, s>>>((const T*)x, (const TW*)w, (const TW*)b, (T*)y, mean, rstd, \
                                                 rows, D, eps, pl.KR, pl.S, gbh::status_ptr());          \
        rc = 0;                                                                                          \
      }                                                                                                  \
    }
    GB_PIPE_DISPATCH(GB_FWDP)
#undef GB_FWDP
    if (rc == 0) {
      GB_CUDA_OK(cudaGetLastError());
      return gbh::E_OK;
    }
  }
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

// Launches the pipelined backward; returns 1 when no plan fits (the caller falls back).
template <typename T, typename TW, typename TS, bool RMS, bool RES>
int norm_bwd_pipe_launch(const void* x, const void* dy, const void* dres, const void* w, const float* mean,
                         const float* rstd, void* dx, void* dgamma, void* dbeta, void* dsum, int dsum_acc,
                         float* part, int part_rows, long long rows, int D, cudaStream_t s) {
  constexpr int V = IO<T>::V;
  constexpr int NP = RES ? 3 : 2;
  const int nvec = D / V;
  const bool want_param = dgamma != nullptr || dbeta != nullptr || (RES && dsum != nullptr);
  int grid = 0, rc = 1;
#define GB_BWDP(G, VPT)                                                                                  \
    {                                                                                                    \
      constexpr int NGc = kPipeConsumers / G;                                                            \
      PipePlan pl = pipe_plan((size_t)D * sizeof(T), NGc, NP, (size_t)D * sizeof(float),                    \
                              want_param ? (size_t)NGc * NP * D * sizeof(float) : 0);                    \
      if (pl.ok) {                                                                                       \
        auto kern = norm_bwd_pipe_kernel<T, TW, G, VPT, RMS, RES>;                                       \
        static bool attr_set = false;                                                                    \
        if (!attr_set) {                                                                                 \
          GB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024)); \
          attr_set = true;                                                                               \
        }                                                                                                \
        const long long ntiles = (rows + NGc * pl.KR - 1) / (NGc * pl.KR);                               \
        grid = (int)(ntiles < 296 ? ntiles : 296);                                                       \
        if (want_param && grid > part_rows) grid = part_rows;                                            \
        kern<<<grid, kPipeThreads, pl.smem, s>>>((const T*)x, (const T*)dy, (const T*)dres, (const TW*)w, mean, \
                                                 rstd, (T*)dx, want_param ? part : nullptr, rows, D, pl.KR, \
                                                 pl.S, gbh::status_ptr());                               \
        rc = 0;                                                                                          \
      }                                                                                                  \
    }
  GB_PIPE_DISPATCH_RES(GB_BWDP)
#undef GB_BWDP
  if (rc != 0) return 1;
  GB_CUDA_OK(cudaGetLastError());
  if (want_param) {
    norm_param_reduce_kernel<TW, TS><<<(NP * D + 31) / 32, dim3(32, 32), 0, s>>>(
        part, grid, D, NP, (TW*)dgamma, (TW*)dbeta, (TS*)dsum, dsum_acc);
    GB_CUDA_OK(cudaGetLastError());
  }
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
  if (g_norm_pipe && !(want_param && (part == nullptr || part_rows < 1))) {
    const int rc = norm_bwd_pipe_launch<T, TW, float, RMS, false>(x, dy, nullptr, w, mean, rstd, dx, dgamma, dbeta,
                                                                  nullptr, 0, part, part_rows, rows, D, s);
    if (rc <= 0) return rc;
  }
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
    norm_param_reduce_kernel<TW, float><<<(2 * D + 31) / 32, dim3(32, 32), 0, s>>>(
        part, grid, D, 2, (TW*)dgamma, (TW*)dbeta, (float*)nullptr, 0);
    GB_CUDA_OK(cudaGetLastError());
  }
  return gbh::E_OK;
}

}  // namespace

enum { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2 };

// Maximum number of partial rows the backward may use; scratch must hold
// gb_norm_bwd_scratch_rows() * 2 * D floats.
GB_EXPORT int gb_norm_bwd_scratch_rows() { return 148 * 2; }

// pipelined = 1 (default): rows stream through a shared-memory ring filled by bulk copies;
// 0: every warp loads its own rows (kept for comparison and as the fallback).
GB_EXPORT int gb_norm_tune(int pipelined) {
  g_norm_pipe = pipelined != 0;
  return gbh::E_OK;
}

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
  GB_BOUNDS_BIND();
  GB_BOUNDS_EXTENT(0, scratch_rows, s);
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

// Backward of "norm with a residual bypass": y = norm(x) and x itself both feed later layers,
// so the gradient of x is norm_bwd(dy) + dres.  One pass produces dx = norm_bwd(dy) + dres,
// dgamma / dbeta, and dsum = column sums of dres (written, or added when dsum_accumulate, in
// the input dtype, or fp32 when dsum_f32).  Needs rows of whole 16-byte vectors, at most 1024
// of them, 16-byte aligned pointers, and scratch of scratch_rows * 3 * D floats; returns
// E_BAD_ARG otherwise (callers then run the three steps separately).
GB_EXPORT int gb_norm_bwd_res(int kind, int dtype, int wdtype, const void* x, const void* dy,
                              const void* dres, const void* w, const float* mean, const float* rstd,
                              void* dx, void* dgamma, void* dbeta, void* dsum, int dsum_f32,
                              int dsum_accumulate, float* scratch, int scratch_rows, long long rows,
                              int D, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (rows <= 0 || D <= 0) return gbh::E_OK;
  GB_BOUNDS_BIND();
  GB_BOUNDS_EXTENT(0, scratch_rows, s);
  const int V = dtype == DT_F32 ? 4 : 8;
  const bool aligned = (D % V == 0) && (D / V <= 1024) &&
                       ((((uintptr_t)x | (uintptr_t)dy | (uintptr_t)dres | (uintptr_t)dx) & 15) == 0);
  if (!aligned || dres == nullptr || scratch == nullptr || scratch_rows < 1) {
    gbh::set_error("gb_norm_bwd_res: needs aligned rows of at most 1024 vectors, dres and scratch");
    return gbh::E_BAD_ARG;
  }
  int rc = 1;
#define GB_N(DTI, T, WDI, TW)                                                                            \
  if (dtype == DTI && wdtype == WDI) {                                                                   \
    if (dsum_f32)                                                                                        \
      rc = kind ? norm_bwd_pipe_launch<T, TW, float, true, true>(x, dy, dres, w, mean, rstd, dx, dgamma, dbeta,  \
                                                                 dsum, dsum_accumulate, scratch, scratch_rows, rows, D, s) \
                : norm_bwd_pipe_launch<T, TW, float, false, true>(x, dy, dres, w, mean, rstd, dx, dgamma, dbeta, \
                                                                  dsum, dsum_accumulate, scratch, scratch_rows, rows, D, s); \
    else                                                                                                 \
      rc = kind ? norm_bwd_pipe_launch<T, TW, T, true, true>(x, dy, dres, w, mean, rstd, dx, dgamma, dbeta,      \
                                                             dsum, dsum_accumulate, scratch, scratch_rows, rows, D, s) \
                : norm_bwd_pipe_launch<T, TW, T, false, true>(x, dy, dres, w, mean, rstd, dx, dgamma, dbeta,     \
                                                              dsum, dsum_accumulate, scratch, scratch_rows, rows, D, s); \
  }
  GB_N(DT_BF16, __nv_bfloat16, DT_BF16, __nv_bfloat16)
  GB_N(DT_BF16, __nv_bfloat16, DT_F32, float)
  GB_N(DT_F16, __half, DT_F16, __half)
  GB_N(DT_F16, __half, DT_F32, float)
  GB_N(DT_F32, float, DT_F32, float)
#undef GB_N
  if (rc == 1) {
    gbh::set_error("gb_norm_bwd_res: no kernel plan for dtype pair %d/%d, D %d", dtype, wdtype, D);
    return gbh::E_BAD_ARG;
  }
  return rc;
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
