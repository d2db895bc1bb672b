// Elementwise engine: every unary op of the registry (forward and backward on
// the device), parameterised activations, binary add/sub/mul/div with stride-0
// broadcasting, casts, and fills.  bf16 / fp16 / fp32 compute in fp32; fp64 in
// fp64.  Contiguous, 16-byte aligned tensors take the 128-bit vector path.
//
// The reference registers the same op set on the host (tensor/ops_unary.go,
// tensor/ops_activation.go) and runs only 12 of them as fp64 kernels, forward
// only (backend/cuda/gonn_cuda.cu:82-109); backward always ran on the host
// (tensor/registry.go:77-83).
#include "common.cuh"

using namespace gb;

namespace {

// Op ids: keep in sync with gonn_b200/ops/elementwise.py
enum UnaryOp : int {
  U_EXP = 0, U_LOG, U_SQRT, U_SIN, U_COS, U_TAN, U_ABS, U_RECIPROCAL, U_SQUARE,
  U_RELU, U_SELU, U_SIGMOID, U_TANH, U_HARDTANH, U_HARDSIGMOID, U_SOFTPLUS, U_SOFTSIGN,
  U_GELU, U_GELUEXACT, U_SILU, U_HARDSWISH, U_MISH, U_RELU6, U_LOGSIGMOID, U_TANHSHRINK,
  U_POW, U_CLIP, U_LEAKYRELU, U_ELU, U_HARDSHRINK, U_SOFTSHRINK, U_SOFTPLUSBETA, U_THRESHOLD,
  U_CELU, U_NEG, U_SCALE_ADD /* p0*x + p1 */, U_COUNT
};
enum BinaryOp : int { B_ADD = 0, B_SUB, B_MUL, B_DIV, B_COUNT };

template <typename CT> __device__ __forceinline__ CT t_exp(CT x);
template <> __device__ __forceinline__ float t_exp<float>(float x) { return __expf(x); }
template <> __device__ __forceinline__ double t_exp<double>(double x) { return exp(x); }
template <typename CT> __device__ __forceinline__ CT t_tanh(CT x);
template <> __device__ __forceinline__ float t_tanh<float>(float x) { return tanhf(x); }
template <> __device__ __forceinline__ double t_tanh<double>(double x) { return tanh(x); }

template <typename CT>
__device__ __forceinline__ CT sigmoid_(CT x) { return CT(1) / (CT(1) + t_exp<CT>(-x)); }
template <typename CT>
__device__ __forceinline__ CT softplus_(CT x) { return x > CT(20) ? x : (CT)log1p((double)0 + t_exp<CT>(x)); }
template <>
__device__ __forceinline__ float softplus_<float>(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

// forward value
template <typename CT>
__device__ __forceinline__ CT ufwd(int op, CT x, CT p0, CT p1) {
  switch (op) {
    case U_EXP: return t_exp<CT>(x);
    case U_LOG: return (CT)log(x);
    case U_SQRT: return (CT)sqrt(x);
    case U_SIN: return (CT)sin(x);
    case U_COS: return (CT)cos(x);
    case U_TAN: return (CT)tan(x);
    case U_ABS: return x < CT(0) ? -x : x;
    case U_RECIPROCAL: return CT(1) / x;
    case U_SQUARE: return x * x;
    case U_RELU: return x > CT(0) ? x : CT(0);
    case U_SELU: {
      const CT a = CT(1.6732632423543772848170429916717), s = CT(1.0507009873554804934193349852946);
      return x > CT(0) ? s * x : s * a * (t_exp<CT>(x) - CT(1));
    }
    case U_SIGMOID: return sigmoid_<CT>(x);
    case U_TANH: return t_tanh<CT>(x);
    case U_HARDTANH: return x < CT(-1) ? CT(-1) : (x > CT(1) ? CT(1) : x);
    case U_HARDSIGMOID: {
      CT v = x / CT(6) + CT(0.5);
      return v < CT(0) ? CT(0) : (v > CT(1) ? CT(1) : v);
    }
    case U_SOFTPLUS: return softplus_<CT>(x);
    case U_SOFTSIGN: return x / (CT(1) + (x < CT(0) ? -x : x));
    case U_GELU: {
      const CT k0 = CT(0.7978845608028654), k1 = CT(0.044715);
      return CT(0.5) * x * (CT(1) + t_tanh<CT>(k0 * (x + k1 * x * x * x)));
    }
    case U_GELUEXACT: return CT(0.5) * x * (CT(1) + (CT)erf(x * CT(0.7071067811865476)));
    case U_SILU: return x * sigmoid_<CT>(x);
    case U_HARDSWISH: {
      CT r = x + CT(3);
      r = r < CT(0) ? CT(0) : (r > CT(6) ? CT(6) : r);
      return x * r / CT(6);
    }
    case U_MISH: return x * t_tanh<CT>(softplus_<CT>(x));
    case U_RELU6: return x < CT(0) ? CT(0) : (x > CT(6) ? CT(6) : x);
    case U_LOGSIGMOID: return -softplus_<CT>(-x);
    case U_TANHSHRINK: return x - t_tanh<CT>(x);
    case U_POW: return (CT)pow(x, p0);
    case U_CLIP: return x < p0 ? p0 : (x > p1 ? p1 : x);
    case U_LEAKYRELU: return x > CT(0) ? x : p0 * x;
    case U_ELU: return x > CT(0) ? x : p0 * (t_exp<CT>(x) - CT(1));
    case U_HARDSHRINK: return (x > p0 || x < -p0) ? x : CT(0);
    case U_SOFTSHRINK: return x > p0 ? x - p0 : (x < -p0 ? x + p0 : CT(0));
    case U_SOFTPLUSBETA: {
      CT bx = p0 * x;
      return bx > p1 ? x : (CT)log1p((double)t_exp<CT>(bx)) / p0;
    }
    case U_THRESHOLD: return x > p0 ? x : p1;
    case U_CELU: {
      CT neg = p0 * (t_exp<CT>(x / p0) - CT(1));
      return (x > CT(0) ? x : CT(0)) + (neg < CT(0) ? neg : CT(0));
    }
    case U_NEG: return -x;
    case U_SCALE_ADD: return p0 * x + p1;
  }
  return x;
}

// derivative d f / d x evaluated at x
template <typename CT>
__device__ __forceinline__ CT ubwd(int op, CT x, CT p0, CT p1) {
  switch (op) {
    case U_EXP: return t_exp<CT>(x);
    case U_LOG: return CT(1) / x;
    case U_SQRT: return CT(0.5) / (CT)sqrt(x);
    case U_SIN: return (CT)cos(x);
    case U_COS: return -(CT)sin(x);
    case U_TAN: { CT c = (CT)cos(x); return CT(1) / (c * c); }
    case U_ABS: return x > CT(0) ? CT(1) : (x < CT(0) ? CT(-1) : CT(0));
    case U_RECIPROCAL: return CT(-1) / (x * x);
    case U_SQUARE: return CT(2) * x;
    case U_RELU: return x > CT(0) ? CT(1) : CT(0);
    case U_SELU: {
      const CT a = CT(1.6732632423543772848170429916717), s = CT(1.0507009873554804934193349852946);
      return x > CT(0) ? s : s * a * t_exp<CT>(x);
    }
    case U_SIGMOID: { CT s = sigmoid_<CT>(x); return s * (CT(1) - s); }
    case U_TANH: { CT t = t_tanh<CT>(x); return CT(1) - t * t; }
    case U_HARDTANH: return (x > CT(-1) && x < CT(1)) ? CT(1) : CT(0);
    case U_HARDSIGMOID: return (x > CT(-3) && x < CT(3)) ? CT(1) / CT(6) : CT(0);
    case U_SOFTPLUS: return x > CT(20) ? CT(1) : sigmoid_<CT>(x);
    case U_SOFTSIGN: { CT d = CT(1) + (x < CT(0) ? -x : x); return CT(1) / (d * d); }
    case U_GELU: {
      const CT k0 = CT(0.7978845608028654), k1 = CT(0.044715);
      CT t = t_tanh<CT>(k0 * (x + k1 * x * x * x));
      return CT(0.5) * (CT(1) + t) + CT(0.5) * x * (CT(1) - t * t) * k0 * (CT(1) + CT(3) * k1 * x * x);
    }
    case U_GELUEXACT:
      return CT(0.5) * (CT(1) + (CT)erf(x * CT(0.7071067811865476))) +
             x * CT(0.3989422804014327) * t_exp<CT>(CT(-0.5) * x * x);
    case U_SILU: { CT s = sigmoid_<CT>(x); return s * (CT(1) + x * (CT(1) - s)); }
    case U_HARDSWISH: return x < CT(-3) ? CT(0) : (x > CT(3) ? CT(1) : (CT(2) * x + CT(3)) / CT(6));
    case U_MISH: {
      CT t = t_tanh<CT>(softplus_<CT>(x));
      return t + x * (CT(1) - t * t) * sigmoid_<CT>(x);
    }
    case U_RELU6: return (x > CT(0) && x < CT(6)) ? CT(1) : CT(0);
    case U_LOGSIGMOID: return sigmoid_<CT>(-x);
    case U_TANHSHRINK: { CT t = t_tanh<CT>(x); return t * t; }
    case U_POW: return p0 * (CT)pow(x, p0 - CT(1));
    case U_CLIP: return (x >= p0 && x <= p1) ? CT(1) : CT(0);
    case U_LEAKYRELU: return x > CT(0) ? CT(1) : p0;
    case U_ELU: return x > CT(0) ? CT(1) : p0 * t_exp<CT>(x);
    case U_HARDSHRINK: return (x > p0 || x < -p0) ? CT(1) : CT(0);
    case U_SOFTSHRINK: return (x > p0 || x < -p0) ? CT(1) : CT(0);
    case U_SOFTPLUSBETA: return p0 * x > p1 ? CT(1) : sigmoid_<CT>(p0 * x);
    case U_THRESHOLD: return x > p0 ? CT(1) : CT(0);
    case U_CELU: return x > CT(0) ? CT(1) : t_exp<CT>(x / p0);
    case U_NEG: return CT(-1);
    case U_SCALE_ADD: return p0;
  }
  return CT(1);
}

template <typename T> struct Conv;
template <> struct Conv<float> {
  using CT = float;
  static __device__ __forceinline__ float ld(float v) { return v; }
  static __device__ __forceinline__ float st(float v) { return v; }
};
template <> struct Conv<double> {
  using CT = double;
  static __device__ __forceinline__ double ld(double v) { return v; }
  static __device__ __forceinline__ double st(double v) { return v; }
};
template <> struct Conv<__nv_bfloat16> {
  using CT = float;
  static __device__ __forceinline__ float ld(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 st(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Conv<__half> {
  using CT = float;
  static __device__ __forceinline__ float ld(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half st(float v) { return __float2half_rn(v); }
};

template <typename T, int N>
struct alignas(sizeof(T) * N) Vec { T v[N]; };

// MODE 0: y = f(x); MODE 1: dx = dy * f'(x)
template <typename T, int MODE, int OP>
__global__ void unary_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ y,
                             long long n, int vec_ok, double p0d, double p1d) {
  using CT = typename Conv<T>::CT;
  constexpr int V = 16 / sizeof(T);
  const CT p0 = (CT)p0d, p1 = (CT)p1d;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  long long done = 0;
  if (vec_ok) {
    const long long nv = n / V;
    const Vec<T, V>* xv = reinterpret_cast<const Vec<T, V>*>(x);
    const Vec<T, V>* dv = reinterpret_cast<const Vec<T, V>*>(dy);
    Vec<T, V>* yv = reinterpret_cast<Vec<T, V>*>(y);
    for (long long i = tid; i < nv; i += nth) {
      Vec<T, V> a = xv[i], o, g;
      if (MODE == 1) g = dv[i];
#pragma unroll
      for (int j = 0; j < V; j++) {
        CT xv_ = Conv<T>::ld(a.v[j]);
        CT r = MODE == 0 ? ufwd<CT>(OP, xv_, p0, p1) : Conv<T>::ld(g.v[j]) * ubwd<CT>(OP, xv_, p0, p1);
        o.v[j] = Conv<T>::st(r);
      }
      yv[i] = o;
    }
    done = nv * V;
  }
  for (long long i = done + tid; i < n; i += nth) {
    CT xv_ = Conv<T>::ld(x[i]);
    CT r = MODE == 0 ? ufwd<CT>(OP, xv_, p0, p1) : Conv<T>::ld(dy[i]) * ubwd<CT>(OP, xv_, p0, p1);
    y[i] = Conv<T>::st(r);
  }
}

template <typename CT>
__device__ __forceinline__ CT bin(int op, CT a, CT b) {
  switch (op) {
    case B_ADD: return a + b;
    case B_SUB: return a - b;
    case B_MUL: return a * b;
    default: return a / b;
  }
}

template <typename T, int OP>
__global__ void binary_same_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ c,
                                   long long n, int vec_ok) {
  using CT = typename Conv<T>::CT;
  constexpr int V = 16 / sizeof(T);
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  long long done = 0;
  if (vec_ok) {
    const long long nv = n / V;
    const Vec<T, V>* av = reinterpret_cast<const Vec<T, V>*>(a);
    const Vec<T, V>* bv = reinterpret_cast<const Vec<T, V>*>(b);
    Vec<T, V>* cv = reinterpret_cast<Vec<T, V>*>(c);
    for (long long i = tid; i < nv; i += nth) {
      Vec<T, V> x = av[i], y = bv[i], o;
#pragma unroll
      for (int j = 0; j < V; j++) o.v[j] = Conv<T>::st(bin<CT>(OP, Conv<T>::ld(x.v[j]), Conv<T>::ld(y.v[j])));
      cv[i] = o;
    }
    done = nv * V;
  }
  for (long long i = done + tid; i < n; i += nth)
    c[i] = Conv<T>::st(bin<CT>(OP, Conv<T>::ld(a[i]), Conv<T>::ld(b[i])));
}

struct BcastDims {
  int rank;
  long long shape[6];
  long long sa[6];
  long long sb[6];
};

// Broadcasting binary op: output is contiguous, inputs are addressed through
// strides in which a broadcast dimension has stride 0 (nothing is materialised).
template <typename T, int OP>
__global__ void binary_bcast_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ c,
                                    long long n, BcastDims d) {
  using CT = typename Conv<T>::CT;
  const long long nth = (long long)gridDim.x * blockDim.x;
  if (n <= 0x7fffffffLL) {
    // 32-bit index arithmetic: a 64-bit division per dimension per element dominates otherwise
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += nth) {
      unsigned r = (unsigned)i;
      long long oa = 0, ob = 0;
#pragma unroll
      for (int k = 5; k >= 0; k--) {
        if (k < d.rank) {
          const unsigned sh = (unsigned)d.shape[k];
          const unsigned q = r / sh;
          const unsigned idx = r - q * sh;
          r = q;
          oa += idx * d.sa[k];
          ob += idx * d.sb[k];
        }
      }
      c[i] = Conv<T>::st(bin<CT>(OP, Conv<T>::ld(a[oa]), Conv<T>::ld(b[ob])));
    }
    return;
  }
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += nth) {
    long long r = i, oa = 0, ob = 0;
#pragma unroll
    for (int k = 5; k >= 0; k--) {
      if (k < d.rank) {
        long long idx = r % d.shape[k];
        r /= d.shape[k];
        oa += idx * d.sa[k];
        ob += idx * d.sb[k];
      }
    }
    c[i] = Conv<T>::st(bin<CT>(OP, Conv<T>::ld(a[oa]), Conv<T>::ld(b[ob])));
  }
}

// The commonest broadcast: one operand is contiguous over the whole output, the other repeats along
// the leading dimensions and is contiguous over the trailing `inner` elements (a bias row, a position
// table added to every batch entry).  16-byte accesses on both; SWAP: the repeating operand is the
// left one (matters for sub / div).  Needs inner % V == 0 and 16-byte aligned pointers.
template <typename T, int OP, bool SWAP>
__global__ void binary_rowvec_kernel(const T* __restrict__ full, const T* __restrict__ row, T* __restrict__ c,
                                     long long nvec, long long inner_vec) {
  using CT = typename Conv<T>::CT;
  constexpr int V = 16 / sizeof(T);
  const Vec<T, V>* fv = reinterpret_cast<const Vec<T, V>*>(full);
  const Vec<T, V>* rv = reinterpret_cast<const Vec<T, V>*>(row);
  Vec<T, V>* cv = reinterpret_cast<Vec<T, V>*>(c);
  const long long nth = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += nth) {
    const long long j = nvec <= 0x7fffffffLL ? (long long)((unsigned)i % (unsigned)inner_vec) : i % inner_vec;
    const Vec<T, V> x = fv[i], y = rv[j];
    Vec<T, V> o;
#pragma unroll
    for (int k = 0; k < V; k++) {
      const CT xa = Conv<T>::ld(x.v[k]), yb = Conv<T>::ld(y.v[k]);
      o.v[k] = Conv<T>::st(SWAP ? bin<CT>(OP, yb, xa) : bin<CT>(OP, xa, yb));
    }
    cv[i] = o;
  }
}

// Is operand `s` (strides) contiguous over the whole shape?  And does operand `s` repeat (stride 0)
// over dims [0, j) and run contiguously over dims [j, rank)?  Returns that j, or -1.
inline bool bcast_full(const BcastDims& d, const long long* s) {
  long long want = 1;
  for (int k = d.rank - 1; k >= 0; k--) {
    if (d.shape[k] != 1 && s[k] != want) return false;
    want *= d.shape[k];
  }
  return true;
}
inline int bcast_row_split(const BcastDims& d, const long long* s) {
  long long want = 1;
  int k = d.rank - 1;
  for (; k >= 0; k--) {
    if (d.shape[k] == 1) { continue; }
    if (s[k] != want) break;
    want *= d.shape[k];
  }
  for (int q = k; q >= 0; q--)
    if (d.shape[q] != 1 && s[q] != 0) return -1;
  return k + 1;
}

template <typename TI, typename TO>
__global__ void cast_kernel(const TI* __restrict__ x, TO* __restrict__ y, long long n) {
  const long long nth = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += nth) {
    double v = (double)Conv<TI>::ld(x[i]);
    y[i] = Conv<TO>::st((typename Conv<TO>::CT)v);
  }
}

inline int grid_for(long long work, int block, int max_blocks = 148 * 16) {
  long long g = (work + block - 1) / block;
  if (g < 1) g = 1;
  if (g > max_blocks) g = max_blocks;
  return (int)g;
}

template <typename T, int MODE>
int launch_unary(int op, const void* x, const void* dy, void* y, long long n, double p0, double p1,
                 cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  int vec_ok = (((uintptr_t)x | (uintptr_t)y | (uintptr_t)dy) & 15) == 0;
  int grid = grid_for((n + V - 1) / V, 256);
#define GB_U(OPID)                                                                            \
  case OPID:                                                                                  \
    unary_kernel<T, MODE, OPID><<<grid, 256, 0, s>>>((const T*)x, (const T*)dy, (T*)y, n, vec_ok, p0, p1); \
    break;
  switch (op) {
    GB_U(U_EXP) GB_U(U_LOG) GB_U(U_SQRT) GB_U(U_SIN) GB_U(U_COS) GB_U(U_TAN) GB_U(U_ABS)
    GB_U(U_RECIPROCAL) GB_U(U_SQUARE) GB_U(U_RELU) GB_U(U_SELU) GB_U(U_SIGMOID) GB_U(U_TANH)
    GB_U(U_HARDTANH) GB_U(U_HARDSIGMOID) GB_U(U_SOFTPLUS) GB_U(U_SOFTSIGN) GB_U(U_GELU)
    GB_U(U_GELUEXACT) GB_U(U_SILU) GB_U(U_HARDSWISH) GB_U(U_MISH) GB_U(U_RELU6) GB_U(U_LOGSIGMOID)
    GB_U(U_TANHSHRINK) GB_U(U_POW) GB_U(U_CLIP) GB_U(U_LEAKYRELU) GB_U(U_ELU) GB_U(U_HARDSHRINK)
    GB_U(U_SOFTSHRINK) GB_U(U_SOFTPLUSBETA) GB_U(U_THRESHOLD) GB_U(U_CELU) GB_U(U_NEG)
    GB_U(U_SCALE_ADD)
    default:
      gbh::set_error("unknown unary op id %d", op);
      return gbh::E_BAD_ARG;
  }
#undef GB_U
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

template <typename T>
int launch_binary(int op, const void* a, const void* b, void* c, long long n, const BcastDims* d,
                  cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  // row-vector broadcast (see binary_rowvec_kernel): 1 = b repeats, 2 = a repeats
  int rv_mode = 0;
  long long rv_inner = 0;
  if (d != nullptr && ((((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15) == 0)) {
    for (int side = 1; side <= 2 && rv_mode == 0; side++) {
      const long long* sf = side == 1 ? d->sa : d->sb;
      const long long* sr = side == 1 ? d->sb : d->sa;
      if (!bcast_full(*d, sf)) continue;
      const int j = bcast_row_split(*d, sr);
      if (j <= 0) continue;                       // -1: no such split; 0: nothing repeats
      long long inner = 1;
      for (int k = j; k < d->rank; k++) inner *= d->shape[k];
      if (inner % V == 0 && n % V == 0 && inner >= V) { rv_mode = side; rv_inner = inner; }
    }
  }
#define GB_B(OPID)                                                                                 \
  case OPID:                                                                                       \
    if (d == nullptr) {                                                                            \
      int vec_ok = (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15) == 0;                       \
      binary_same_kernel<T, OPID><<<grid_for((n + V - 1) / V, 256), 256, 0, s>>>((const T*)a, (const T*)b, (T*)c, n, vec_ok); \
    } else if (rv_mode == 1) {                                                                     \
      binary_rowvec_kernel<T, OPID, false><<<grid_for(n / V, 256), 256, 0, s>>>((const T*)a, (const T*)b, (T*)c, n / V, rv_inner / V); \
    } else if (rv_mode == 2) {                                                                     \
      binary_rowvec_kernel<T, OPID, true><<<grid_for(n / V, 256), 256, 0, s>>>((const T*)b, (const T*)a, (T*)c, n / V, rv_inner / V); \
    } else {                                                                                       \
      binary_bcast_kernel<T, OPID><<<grid_for(n, 256), 256, 0, s>>>((const T*)a, (const T*)b, (T*)c, n, *d); \
    }                                                                                              \
    break;
  switch (op) {
    GB_B(B_ADD) GB_B(B_SUB) GB_B(B_MUL) GB_B(B_DIV)
    default:
      gbh::set_error("unknown binary op id %d", op);
      return gbh::E_BAD_ARG;
  }
#undef GB_B
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

}  // namespace

enum { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2, DT_F64 = 3 };

// y = f(x) for the op id `op` with parameters p0, p1.
GB_EXPORT int gb_unary_fwd(int op, int dtype, const void* x, void* y, long long n, double p0,
                           double p1, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (n <= 0) return gbh::E_OK;
  switch (dtype) {
    case DT_BF16: return launch_unary<__nv_bfloat16, 0>(op, x, nullptr, y, n, p0, p1, s);
    case DT_F16: return launch_unary<__half, 0>(op, x, nullptr, y, n, p0, p1, s);
    case DT_F32: return launch_unary<float, 0>(op, x, nullptr, y, n, p0, p1, s);
    case DT_F64: return launch_unary<double, 0>(op, x, nullptr, y, n, p0, p1, s);
  }
  gbh::set_error("gb_unary_fwd: bad dtype %d", dtype);
  return gbh::E_BAD_ARG;
}

// dx = dy * f'(x)
GB_EXPORT int gb_unary_bwd(int op, int dtype, const void* x, const void* dy, void* dx, long long n,
                           double p0, double p1, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (n <= 0) return gbh::E_OK;
  switch (dtype) {
    case DT_BF16: return launch_unary<__nv_bfloat16, 1>(op, x, dy, dx, n, p0, p1, s);
    case DT_F16: return launch_unary<__half, 1>(op, x, dy, dx, n, p0, p1, s);
    case DT_F32: return launch_unary<float, 1>(op, x, dy, dx, n, p0, p1, s);
    case DT_F64: return launch_unary<double, 1>(op, x, dy, dx, n, p0, p1, s);
  }
  gbh::set_error("gb_unary_bwd: bad dtype %d", dtype);
  return gbh::E_BAD_ARG;
}

// c = a (op) b.  rank == 0: same-shape contiguous operands.  Otherwise the
// output is contiguous with `shape`, and sa / sb are the element strides of
// a / b per output dimension (0 where the operand is broadcast).
GB_EXPORT int gb_binary(int op, int dtype, const void* a, const void* b, void* c, long long n,
                        int rank, const long long* shape, const long long* sa,
                        const long long* sb, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (n <= 0) return gbh::E_OK;
  BcastDims d;
  const BcastDims* dp = nullptr;
  if (rank > 0) {
    if (rank > 6) {
      gbh::set_error("gb_binary: at most 6 broadcast dimensions");
      return gbh::E_BAD_ARG;
    }
    d.rank = rank;
    for (int i = 0; i < rank; i++) {
      d.shape[i] = shape[i];
      d.sa[i] = sa[i];
      d.sb[i] = sb[i];
    }
    dp = &d;
  }
  switch (dtype) {
    case DT_BF16: return launch_binary<__nv_bfloat16>(op, a, b, c, n, dp, s);
    case DT_F16: return launch_binary<__half>(op, a, b, c, n, dp, s);
    case DT_F32: return launch_binary<float>(op, a, b, c, n, dp, s);
    case DT_F64: return launch_binary<double>(op, a, b, c, n, dp, s);
  }
  gbh::set_error("gb_binary: bad dtype %d", dtype);
  return gbh::E_BAD_ARG;
}

// Casts between bf16 / fp16 / fp32 / fp64 with round-to-nearest-even.
GB_EXPORT int gb_cast(int src_dtype, int dst_dtype, const void* x, void* y, long long n,
                      void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (n <= 0) return gbh::E_OK;
  int grid = grid_for(n, 256);
#define GB_C(SI, ST, DI, DT_)                                                              \
  if (src_dtype == SI && dst_dtype == DI) {                                                \
    cast_kernel<ST, DT_><<<grid, 256, 0, s>>>((const ST*)x, (DT_*)y, n);                   \
    GB_CUDA_OK(cudaGetLastError());                                                        \
    return gbh::E_OK;                                                                      \
  }
#define GB_CROW(SI, ST)                                                                    \
  GB_C(SI, ST, DT_BF16, __nv_bfloat16) GB_C(SI, ST, DT_F16, __half) GB_C(SI, ST, DT_F32, float) \
  GB_C(SI, ST, DT_F64, double)
  GB_CROW(DT_BF16, __nv_bfloat16) GB_CROW(DT_F16, __half) GB_CROW(DT_F32, float) GB_CROW(DT_F64, double)
#undef GB_CROW
#undef GB_C
  gbh::set_error("gb_cast: bad dtype pair %d -> %d", src_dtype, dst_dtype);
  return gbh::E_BAD_ARG;
}
