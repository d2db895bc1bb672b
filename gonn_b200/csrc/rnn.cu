// Fused gate arithmetic of the LSTM and GRU cells, forward and backward.
//
// The reference unrolls every time step into the tape as two Linear layers plus a handful
// of elementwise nodes per gate (nn/rnn.go:159-286: LSTM gate order i, f, g, o with
// c' = f*c + i*g, h' = o*tanh(c'); GRU gates r, z, n with n = tanh(xn + r*hn),
// h' = (1-z)*n + z*h).  Here the two GEMMs stay GEMMs and everything between them and the
// new state is one kernel per direction: one read of the gate pre-activations, one write of
// the state (and of the activated gates the backward needs).
#include "common.cuh"

using namespace gb;

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p, long long i) { return (float)p[i]; }
__device__ __forceinline__ float sigm(float x) { return 1.f / (1.f + __expf(-x)); }

// gates: (B, 4H) pre-activations (x W_ih^T + b + h W_hh^T); c: (B, H).
// act: (B, 4H) receives the activated gates (i, f, g, o) for the backward.
template <typename T>
__global__ void lstm_fwd_kernel(const T* __restrict__ gates, const T* __restrict__ c, T* __restrict__ h_new,
                                T* __restrict__ c_new, T* __restrict__ act, long long B, int H) {
  const long long total = B * H;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long b = i / H;
    const int j = (int)(i - b * H);
    const T* g = gates + b * 4 * H;
    const float ig = sigm(ldf(g, j)), fg = sigm(ldf(g, H + j));
    const float gg = tanhf(ldf(g, 2 * H + j)), og = sigm(ldf(g, 3 * H + j));
    const float cn = fg * ldf(c, i) + ig * gg;
    c_new[i] = (T)cn;
    h_new[i] = (T)(og * tanhf(cn));
    T* a = act + b * 4 * H;
    a[j] = (T)ig; a[H + j] = (T)fg; a[2 * H + j] = (T)gg; a[3 * H + j] = (T)og;
  }
}

// dgates (B, 4H) and dc_prev (B, H) from dh', dc' (either may be null = zeros).
template <typename T>
__global__ void lstm_bwd_kernel(const T* __restrict__ act, const T* __restrict__ c, const T* __restrict__ c_new,
                                const T* __restrict__ dh, const T* __restrict__ dc, T* __restrict__ dgates,
                                T* __restrict__ dc_prev, long long B, int H) {
  const long long total = B * H;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long b = i / H;
    const int j = (int)(i - b * H);
    const T* a = act + b * 4 * H;
    const float ig = ldf(a, j), fg = ldf(a, H + j), gg = ldf(a, 2 * H + j), og = ldf(a, 3 * H + j);
    const float tc = tanhf(ldf(c_new, i));
    const float dhv = dh ? ldf(dh, i) : 0.f;
    const float dcv = (dc ? ldf(dc, i) : 0.f) + dhv * og * (1.f - tc * tc);
    T* d = dgates + b * 4 * H;
    d[j] = (T)(dcv * gg * ig * (1.f - ig));
    d[H + j] = (T)(dcv * ldf(c, i) * fg * (1.f - fg));
    d[2 * H + j] = (T)(dcv * ig * (1.f - gg * gg));
    d[3 * H + j] = (T)(dhv * tc * og * (1.f - og));
    dc_prev[i] = (T)(dcv * fg);
  }
}

// xg, hg: (B, 3H) pre-activations of the input and hidden projections (biases included).
// act: (B, 4H) receives r, z, n and hn (the hidden part of the candidate) for the backward.
template <typename T>
__global__ void gru_fwd_kernel(const T* __restrict__ xg, const T* __restrict__ hg, const T* __restrict__ h,
                               T* __restrict__ h_new, T* __restrict__ act, long long B, int H) {
  const long long total = B * H;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long b = i / H;
    const int j = (int)(i - b * H);
    const T* x3 = xg + b * 3 * H;
    const T* h3 = hg + b * 3 * H;
    const float r = sigm(ldf(x3, j) + ldf(h3, j));
    const float z = sigm(ldf(x3, H + j) + ldf(h3, H + j));
    const float hn = ldf(h3, 2 * H + j);
    const float n = tanhf(ldf(x3, 2 * H + j) + r * hn);
    h_new[i] = (T)((1.f - z) * n + z * ldf(h, i));
    T* a = act + b * 4 * H;
    a[j] = (T)r; a[H + j] = (T)z; a[2 * H + j] = (T)n; a[3 * H + j] = (T)hn;
  }
}

// dxg, dhg (B, 3H) and the direct path dh_prev = dh' * z.
template <typename T>
__global__ void gru_bwd_kernel(const T* __restrict__ act, const T* __restrict__ h, const T* __restrict__ dh,
                               T* __restrict__ dxg, T* __restrict__ dhg, T* __restrict__ dh_prev, long long B,
                               int H) {
  const long long total = B * H;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long b = i / H;
    const int j = (int)(i - b * H);
    const T* a = act + b * 4 * H;
    const float r = ldf(a, j), z = ldf(a, H + j), n = ldf(a, 2 * H + j), hn = ldf(a, 3 * H + j);
    const float g = ldf(dh, i);
    const float dn = g * (1.f - z) * (1.f - n * n);   // through tanh
    const float dz = g * (ldf(h, i) - n) * z * (1.f - z);
    const float dr = dn * hn * r * (1.f - r);
    T* dx3 = dxg + b * 3 * H;
    T* dh3 = dhg + b * 3 * H;
    dx3[j] = (T)dr; dx3[H + j] = (T)dz; dx3[2 * H + j] = (T)dn;
    dh3[j] = (T)dr; dh3[H + j] = (T)dz; dh3[2 * H + j] = (T)(dn * r);
    dh_prev[i] = (T)(g * z);
  }
}

inline int grid_for(long long work) {
  long long g = (work + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  return g < 1 ? 1 : (int)g;
}

}  // namespace

enum { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2, DT_F64 = 3 };

#define GB_RNN_DISPATCH(CALL)                                   \
  switch (dtype) {                                              \
    case DT_BF16: { using T = __nv_bfloat16; CALL; } break;     \
    case DT_F16: { using T = __half; CALL; } break;             \
    case DT_F32: { using T = float; CALL; } break;              \
    default:                                                    \
      gbh::set_error("rnn gates: unsupported dtype %d", dtype); \
      return gbh::E_BAD_ARG;                                    \
  }

GB_EXPORT int gb_lstm_gates_fwd(int dtype, const void* gates, const void* c, void* h_new, void* c_new, void* act,
                                long long B, int H, void* stream) {
  if (B * H <= 0) return gbh::E_OK;
  cudaStream_t s = (cudaStream_t)stream;
  GB_RNN_DISPATCH((lstm_fwd_kernel<T><<<grid_for(B * H), 256, 0, s>>>((const T*)gates, (const T*)c, (T*)h_new,
                                                                      (T*)c_new, (T*)act, B, H)));
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

GB_EXPORT int gb_lstm_gates_bwd(int dtype, const void* act, const void* c, const void* c_new, const void* dh,
                                const void* dc, void* dgates, void* dc_prev, long long B, int H, void* stream) {
  if (B * H <= 0) return gbh::E_OK;
  cudaStream_t s = (cudaStream_t)stream;
  GB_RNN_DISPATCH((lstm_bwd_kernel<T><<<grid_for(B * H), 256, 0, s>>>((const T*)act, (const T*)c, (const T*)c_new,
                                                                      (const T*)dh, (const T*)dc, (T*)dgates,
                                                                      (T*)dc_prev, B, H)));
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

GB_EXPORT int gb_gru_gates_fwd(int dtype, const void* xg, const void* hg, const void* h, void* h_new, void* act,
                               long long B, int H, void* stream) {
  if (B * H <= 0) return gbh::E_OK;
  cudaStream_t s = (cudaStream_t)stream;
  GB_RNN_DISPATCH((gru_fwd_kernel<T><<<grid_for(B * H), 256, 0, s>>>((const T*)xg, (const T*)hg, (const T*)h,
                                                                     (T*)h_new, (T*)act, B, H)));
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

GB_EXPORT int gb_gru_gates_bwd(int dtype, const void* act, const void* h, const void* dh, void* dxg, void* dhg,
                               void* dh_prev, long long B, int H, void* stream) {
  if (B * H <= 0) return gbh::E_OK;
  cudaStream_t s = (cudaStream_t)stream;
  GB_RNN_DISPATCH((gru_bwd_kernel<T><<<grid_for(B * H), 256, 0, s>>>((const T*)act, (const T*)h, (const T*)dh,
                                                                     (T*)dxg, (T*)dhg, (T*)dh_prev, B, H)));
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}
