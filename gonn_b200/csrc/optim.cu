// Multi-tensor fused optimizer kernels: SGD (momentum / Nesterov), Adam, AdamW,
// Lion, LAMB (two phases), global gradient norm and scaling.  One launch updates
// up to kMaxTensors tensors; a CTA works on one 4096-element chunk of one
// tensor.  Parameters may be bf16 / fp16 with an fp32 master copy, or fp32 /
// fp64 without one; optimizer state is fp32 (fp64 for fp64 parameters).
//
// Update rules follow the reference's per-element loops: SGD v = mu*v + g,
// Nesterov g + mu*v (optim/sgd.go:47-69); Adam p -= lr*mhat/(sqrt(vhat)+eps)
// with eps outside the root and AdamW's p -= lr*wd*p applied first
// (optim/adam.go:61-77, optim/adamw.go:64-84); Lion (optim/lion.go:61-76); LAMB
// trust ratio per tensor with eps 1e-6 (optim/lamb.go:73-108).
#include "common.cuh"

using namespace gb;

namespace {

constexpr int kMaxTensors = 48;
constexpr int kChunk = 4096;
constexpr int kThreads = 256;

struct TensorList {
  int n;
  void* p[kMaxTensors];       // parameter (model dtype)
  void* g[kMaxTensors];       // gradient (model dtype)
  void* master[kMaxTensors];  // fp32 master copy or null
  void* s0[kMaxTensors];      // state 0 (m / momentum)
  void* s1[kMaxTensors];      // state 1 (v) or null
  long long numel[kMaxTensors];
  int chunk_start[kMaxTensors + 1];  // prefix sum of chunk counts
};

struct Hyper {
  float lr, wd, b1, b2, eps, bc1, bc2, momentum, gscale;
  int nesterov, decoupled, has_momentum;
};

enum Algo : int { A_SGD = 0, A_ADAM = 1, A_LION = 2, A_LAMB1 = 3, A_LAMB2 = 4, A_SQNORM = 5, A_SCALE = 6 };

template <typename T> struct Num { using CT = float; };
template <> struct Num<double> { using CT = double; };
__device__ __forceinline__ float t_sqrt(float x) { return sqrtf(x); }
__device__ __forceinline__ double t_sqrt(double x) { return sqrt(x); }

__device__ __forceinline__ int find_tensor(const TensorList& tl, int chunk) {
  int t = 0;
  while (t + 1 < tl.n && tl.chunk_start[t + 1] <= chunk) t++;
  return t;
}

// T: parameter / gradient dtype.  ST: state dtype (float or double).
template <typename T, typename ST, int ALGO>
__global__ void __launch_bounds__(kThreads)
multi_tensor_kernel(const TensorList tl, const Hyper h, float* __restrict__ aux) {
  using CT = typename Num<T>::CT;
  __shared__ float red[32];
  const int t = find_tensor(tl, blockIdx.x);
  const long long base = (long long)(blockIdx.x - tl.chunk_start[t]) * kChunk;
  const long long n = tl.numel[t];
  // The five arrays of one tensor never overlap, so loads of the next elements may pass the stores
  // of this one: with four elements in flight per thread the kernel is bound by DRAM, not by latency.
  T* __restrict__ p = (T*)tl.p[t];
  T* __restrict__ g = (T*)tl.g[t];
  float* __restrict__ master = (float*)tl.master[t];
  ST* __restrict__ s0 = (ST*)tl.s0[t];
  ST* __restrict__ s1 = (ST*)tl.s1[t];
  CT acc0 = 0, acc1 = 0;
  float trust = 1.f;
  if (ALGO == A_LAMB2) {
    float pn = sqrtf(aux[2 * t]), un = sqrtf(aux[2 * t + 1]);
    trust = (pn > 0.f && un > 0.f) ? pn / un : 1.f;
  }
  const int cnt = (int)(n - base < (long long)kChunk ? n - base : (long long)kChunk);
#pragma unroll 4
  for (int k = threadIdx.x; k < cnt; k += kThreads) {
    const long long i = base + k;
    CT gv = ALGO == A_LAMB2 ? CT(0) : (CT)g[i] * (CT)h.gscale;
    CT pv = master ? (CT)master[i] : (CT)p[i];
    if (ALGO == A_SGD) {
      if (h.wd != 0.f) gv += (CT)h.wd * pv;
      CT upd = gv;
      if (h.has_momentum) {
        CT v = (CT)h.momentum * (CT)s0[i] + gv;
        s0[i] = (ST)v;
        upd = h.nesterov ? gv + (CT)h.momentum * v : v;
      }
      pv -= (CT)h.lr * upd;
    } else if (ALGO == A_ADAM) {
      if (h.wd != 0.f) {
        if (h.decoupled) pv -= (CT)h.lr * (CT)h.wd * pv;
        else gv += (CT)h.wd * pv;
      }
      CT m = (CT)h.b1 * (CT)s0[i] + (CT(1) - (CT)h.b1) * gv;
      CT v = (CT)h.b2 * (CT)s1[i] + (CT(1) - (CT)h.b2) * gv * gv;
      s0[i] = (ST)m;
      s1[i] = (ST)v;
      CT mh = m / (CT)h.bc1, vh = v / (CT)h.bc2;
      pv -= (CT)h.lr * mh / (t_sqrt(vh) + (CT)h.eps);
    } else if (ALGO == A_LION) {
      CT m = (CT)s0[i];
      CT c = (CT)h.b1 * m + (CT(1) - (CT)h.b1) * gv;
      CT u = c > CT(0) ? CT(1) : (c < CT(0) ? CT(-1) : CT(0));
      if (h.wd != 0.f) u += (CT)h.wd * pv;
      pv -= (CT)h.lr * u;
      s0[i] = (ST)((CT)h.b2 * m + (CT(1) - (CT)h.b2) * gv);
    } else if (ALGO == A_LAMB1) {
      // phase 1: moments, update direction stored in the gradient buffer, norms
      CT m = (CT)h.b1 * (CT)s0[i] + (CT(1) - (CT)h.b1) * gv;
      CT v = (CT)h.b2 * (CT)s1[i] + (CT(1) - (CT)h.b2) * gv * gv;
      s0[i] = (ST)m;
      s1[i] = (ST)v;
      CT u = (m / (CT)h.bc1) / (t_sqrt(v / (CT)h.bc2) + (CT)h.eps);
      if (h.wd != 0.f) u += (CT)h.wd * pv;
      g[i] = (T)u;
      acc0 += pv * pv;
      acc1 += u * u;
      continue;
    } else if (ALGO == A_LAMB2) {
      pv -= (CT)h.lr * (CT)trust * (CT)g[i];
    } else if (ALGO == A_SQNORM) {
      acc0 += gv * gv;
      continue;
    } else if (ALGO == A_SCALE) {
      g[i] = (T)gv;
      continue;
    }
    if (master) master[i] = (float)pv;
    p[i] = (T)pv;
  }
  if (ALGO == A_LAMB1) {
    float a = block_sum((float)acc0, red);
    float b = block_sum((float)acc1, red);
    if (threadIdx.x == 0) {
      atomicAdd(&aux[2 * t], a);
      atomicAdd(&aux[2 * t + 1], b);
    }
  } else if (ALGO == A_SQNORM) {
    float a = block_sum((float)acc0, red);
    if (threadIdx.x == 0) aux[blockIdx.x] = a;  // per-chunk partials, summed in order by the caller
  }
}

__global__ void sum_partials_kernel(const float* __restrict__ part, int n, float* __restrict__ out,
                                    int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += part[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s : s;
}

template <typename T, typename ST>
int launch_algo(int algo, const TensorList& tl, const Hyper& h, float* aux, cudaStream_t s) {
  const int grid = tl.chunk_start[tl.n];
  if (grid == 0) return gbh::E_OK;
#define GB_A(A)                                                                   \
  case A:                                                                         \
    multi_tensor_kernel<T, ST, A><<<grid, kThreads, 0, s>>>(tl, h, aux);          \
    break;
  switch (algo) {
    GB_A(A_SGD) GB_A(A_ADAM) GB_A(A_LION) GB_A(A_LAMB1) GB_A(A_LAMB2) GB_A(A_SQNORM) GB_A(A_SCALE)
    default:
      gbh::set_error("multi-tensor: unknown algorithm %d", algo);
      return gbh::E_BAD_ARG;
  }
#undef GB_A
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

}  // namespace

enum { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2, DT_F64 = 3 };

GB_EXPORT int gb_mt_max_tensors() { return kMaxTensors; }
GB_EXPORT int gb_mt_chunk() { return kChunk; }

// One multi-tensor launch.  algo: 0 SGD, 1 Adam/AdamW, 2 Lion, 3 LAMB phase 1
// (aux: 2 floats per tensor, zeroed by the caller), 4 LAMB phase 2, 5 squared
// gradient norm (aux: one float per chunk), 6 gradient scaling by gscale.
// hyper: {lr, wd, b1, b2, eps, bc1, bc2, momentum, gscale}; flags: bit 0
// nesterov, bit 1 decoupled weight decay, bit 2 momentum enabled.
GB_EXPORT int gb_multi_tensor(int algo, int dtype, int n, void* const* params, void* const* grads,
                              void* const* masters, void* const* state0, void* const* state1,
                              const long long* numel, const float* hyper, int flags, float* aux,
                              void* stream) {
  if (n < 0 || n > kMaxTensors) {
    gbh::set_error("gb_multi_tensor: %d tensors, at most %d per launch", n, kMaxTensors);
    return gbh::E_BAD_ARG;
  }
  TensorList tl;
  memset(&tl, 0, sizeof(tl));
  tl.n = n;
  int chunks = 0;
  for (int i = 0; i < n; i++) {
    tl.p[i] = params ? params[i] : nullptr;
    tl.g[i] = grads ? grads[i] : nullptr;
    tl.master[i] = masters ? masters[i] : nullptr;
    tl.s0[i] = state0 ? state0[i] : nullptr;
    tl.s1[i] = state1 ? state1[i] : nullptr;
    tl.numel[i] = numel[i];
    tl.chunk_start[i] = chunks;
    chunks += (int)((numel[i] + kChunk - 1) / kChunk);
  }
  tl.chunk_start[n] = chunks;
  Hyper h;
  h.lr = hyper[0]; h.wd = hyper[1]; h.b1 = hyper[2]; h.b2 = hyper[3]; h.eps = hyper[4];
  h.bc1 = hyper[5]; h.bc2 = hyper[6]; h.momentum = hyper[7]; h.gscale = hyper[8];
  h.nesterov = flags & 1; h.decoupled = (flags >> 1) & 1; h.has_momentum = (flags >> 2) & 1;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case DT_BF16: return launch_algo<__nv_bfloat16, float>(algo, tl, h, aux, s);
    case DT_F16: return launch_algo<__half, float>(algo, tl, h, aux, s);
    case DT_F32: return launch_algo<float, float>(algo, tl, h, aux, s);
    case DT_F64: return launch_algo<double, double>(algo, tl, h, aux, s);
  }
  gbh::set_error("gb_multi_tensor: bad dtype %d", dtype);
  return gbh::E_BAD_ARG;
}

// out[0] (+)= sum(part[0..n))
GB_EXPORT int gb_sum_partials(const float* part, int n, float* out, int accumulate, void* stream) {
  sum_partials_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(part, n, out, accumulate);
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}
