// BatchNorm over (N, C, S) tensors (S = product of the spatial dims), training and
// evaluation, with the cross-rank statistics exchange of SyncBatchNorm fused into
// the normalise kernels.
//
// Reference semantics: batch statistics in training (biased variance for the
// normalisation, n/(n-1) for the running variance, momentum 0.1), running
// statistics in evaluation (nn/batchnorm.go:41-86).  SyncBatchNorm packs
// [sum x | sum x^2 | count] and all-reduces it, uses var = E[x^2] - E[x]^2 clamped
// at 0, and in backward all-reduces [sum dy | sum dy*xhat] while keeping the LOCAL
// sums as the weight / bias gradients (distributed/syncbn.go:104-205).
//
// Kernels:
//   bn_partial      per (channel, split) partial sums of (x, x^2) or (dy, dy*xhat)
//   bn_apply        [CTA 0: combine partials in fixed order, exchange with the peers
//                   through their symmetric buffers, publish mean / invstd, update
//                   the running statistics] then every CTA normalises (+ ReLU)
//   bn_bwd_apply    the same structure for dx
// CTA 0 is dispatched first, so the CTAs that wait for its result never wait for a CTA
// that cannot run; its own wait for the peers is bounded.
#include "comm_dev.cuh"

using namespace gb;
using namespace gbc;

namespace {

constexpr int kSplits = 32;
constexpr int kMaxC = 2048;

// partial[c][split][0..1]; mode 0: (x, x^2); mode 1: (dy, dy * xhat)
template <typename T>
__global__ void bn_partial_kernel(const T* __restrict__ a, const T* __restrict__ xin,
                                  const float* __restrict__ mean, const float* __restrict__ invstd,
                                  float* __restrict__ part, int N, int C, long long S, int mode) {
  __shared__ float red[32];
  const int c = blockIdx.x, sp = blockIdx.y;
  const long long per_n = S;
  const long long total = (long long)N * per_n;
  const long long chunk = (total + kSplits - 1) / kSplits;
  const long long lo = sp * chunk, hi = min(lo + chunk, total);
  float s0 = 0.f, s1 = 0.f;
  const float mu = mode ? mean[c] : 0.f, is = mode ? invstd[c] : 0.f;
  for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const long long n = i / per_n, p = i - n * per_n;
    const long long off = (n * C + c) * S + p;
    const float v = (float)a[off];
    if (mode == 0) {
      s0 += v;
      s1 += v * v;
    } else {
      const float xh = ((float)xin[off] - mu) * is;
      s0 += v;
      s1 += v * xh;
    }
  }
  s0 = block_sum(s0, red);
  s1 = block_sum(s1, red);
  if (threadIdx.x == 0) {
    part[((long long)c * kSplits + sp) * 2] = s0;
    part[((long long)c * kSplits + sp) * 2 + 1] = s1;
  }
}

struct BnArgs {
  PeerTable pt;
  int rank, world;
  long long slot_off;  // byte offset of the exchange area inside the symmetric buffer
  unsigned int epoch;
  int N, C;
  long long S;
  float eps, momentum;
  int training, relu;
  const float* part;       // [C][kSplits][2] local partial sums
  float* stats;            // [2C] : mean | invstd   (published for backward too)
  float* sums;             // [2C] : global (sum0 | sum1) / count, scratch for CTA 0
  float* running_mean;     // may be null
  float* running_var;
  const void* w;           // fp32 affine weight / bias, may be null
  const void* b;
  int* ready;              // device flag: epoch value when stats are valid
  int ready_val;
  int* status;
};

// Combines the local partials (fixed order) and, with world > 1, exchanges the 2C+1
// vector with every peer and sums in rank order.  Runs in CTA 0 only.
__device__ void combine_and_exchange(const BnArgs& a, float* out2c, float* count_out, int* sm_flag) {
  const int C = a.C;
  for (int i = threadIdx.x; i < 2 * C; i += blockDim.x) {
    const int c = i % C, which = i / C;
    float s = 0.f;
    for (int sp = 0; sp < kSplits; sp++) s += a.part[((long long)c * kSplits + sp) * 2 + which];
    out2c[i] = s;
  }
  float count = (float)a.N * (float)a.S;
  __syncthreads();
  if (a.world > 1) {
    const int n = 2 * C + 1;
    for (int p = 0; p < a.world; p++) {
      float* slot = (float*)((char*)a.pt.base[p] + a.slot_off) + (long long)a.rank * n;
      for (int i = threadIdx.x; i < 2 * C; i += blockDim.x) slot[i] = out2c[i];
      if (threadIdx.x == 0) slot[2 * C] = count;
    }
    if (!cta_barrier(a.pt, a.rank, a.world, 7, 0, a.epoch, a.status, sm_flag)) {
      *count_out = count;
      return;
    }
    const float* mine = (const float*)((const char*)a.pt.base[a.rank] + a.slot_off);
    for (int i = threadIdx.x; i < 2 * C; i += blockDim.x) {
      float s = 0.f;
      for (int p = 0; p < a.world; p++) s += __ldcg(mine + (long long)p * n + i);
      out2c[i] = s;
    }
    float cs = 0.f;
    for (int p = 0; p < a.world; p++) cs += __ldcg(mine + (long long)p * n + 2 * C);
    count = cs;
    // the slots may be rewritten only after everyone has read them
    cta_barrier(a.pt, a.rank, a.world, 8, 0, a.epoch + 1, a.status, sm_flag);
  }
  *count_out = count;
  __syncthreads();
}

__device__ __forceinline__ bool wait_ready(const BnArgs& a) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) {
    const uint64_t t0 = globaltimer_ns();
    int ok = 1;
    while (*((volatile int*)a.ready) != a.ready_val) {
      if (globaltimer_ns() - t0 > kWaitBudgetNs) {
        set_status(a.status, ST_COMM_TIMEOUT, 77);
        ok = 0;
        break;
      }
    }
    __threadfence();
    ok_flag = ok;
  }
  __syncthreads();
  return ok_flag != 0;
}

template <typename T>
__global__ void __launch_bounds__(256)
bn_apply_kernel(const T* __restrict__ x, T* __restrict__ y, const BnArgs a) {
  __shared__ int sm_flag;
  __shared__ float s_count;
  const int C = a.C;
  if (a.training) {
    if (blockIdx.x == 0) {
      if (threadIdx.x == 0) sm_flag = 0;
      __syncthreads();
      float cnt;
      combine_and_exchange(a, a.sums, &cnt, &sm_flag);
      if (threadIdx.x == 0) s_count = cnt;
      __syncthreads();
      const float n = s_count;
      for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float mean = a.sums[c] / n;
        float var = a.sums[C + c] / n - mean * mean;
        var = var > 0.f ? var : 0.f;
        a.stats[c] = mean;
        a.stats[C + c] = rsqrtf(var + a.eps);
        if (a.running_mean) {
          const float unbiased = n > 1.f ? var * n / (n - 1.f) : var;
          a.running_mean[c] = (1.f - a.momentum) * a.running_mean[c] + a.momentum * mean;
          a.running_var[c] = (1.f - a.momentum) * a.running_var[c] + a.momentum * unbiased;
        }
      }
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) atomicExch(a.ready, a.ready_val);
    }
    if (!wait_ready(a)) return;
  }
  const float* w = (const float*)a.w;
  const float* b = (const float*)a.b;
  const long long total = (long long)a.N * C * a.S;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)((i / a.S) % C);
    float mean, is;
    if (a.training) {
      mean = __ldcg(a.stats + c);
      is = __ldcg(a.stats + C + c);
    } else {
      mean = a.running_mean[c];
      is = rsqrtf(a.running_var[c] + a.eps);
    }
    float v = ((float)x[i] - mean) * is;
    if (w) v *= w[c];
    if (b) v += b[c];
    if (a.relu) v = v > 0.f ? v : 0.f;
    y[i] = (T)v;
  }
}

// dx = w * invstd * (dy - S1/n - xhat * S2/n); dgamma = local S2, dbeta = local S1
template <typename T>
__global__ void __launch_bounds__(256)
bn_bwd_apply_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ dx,
                    float* __restrict__ dgamma, float* __restrict__ dbeta, const BnArgs a) {
  __shared__ int sm_flag;
  __shared__ float s_count;
  const int C = a.C;
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) sm_flag = 0;
    __syncthreads();
    // local sums are the parameter gradients (kept before the exchange)
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
      float s0 = 0.f, s1 = 0.f;
      for (int sp = 0; sp < kSplits; sp++) {
        s0 += a.part[((long long)c * kSplits + sp) * 2];
        s1 += a.part[((long long)c * kSplits + sp) * 2 + 1];
      }
      if (dbeta) dbeta[c] = s0;
      if (dgamma) dgamma[c] = s1;
    }
    float cnt;
    combine_and_exchange(a, a.sums, &cnt, &sm_flag);
    if (threadIdx.x == 0) s_count = cnt;
    __syncthreads();
    const float n = s_count;
    for (int c = threadIdx.x; c < 2 * C; c += blockDim.x) a.sums[c] = a.sums[c] / n;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) atomicExch(a.ready, a.ready_val);
  }
  if (!wait_ready(a)) return;
  const float* w = (const float*)a.w;
  const long long total = (long long)a.N * C * a.S;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)((i / a.S) % C);
    const float mean = a.stats[c], is = a.stats[C + c];
    const float m1 = __ldcg(a.sums + c), m2 = __ldcg(a.sums + C + c);
    const float xh = ((float)x[i] - mean) * is;
    float g = (float)dy[i];
    float v = is * (g - m1 - xh * m2);
    if (w) v *= w[c];
    dx[i] = (T)v;
  }
}

int g_ready_counter = 0;

inline int grid_for(long long work) {
  long long g = (work + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  if (g < 1) g = 1;
  return (int)g;
}

void fill_comm(BnArgs& a, int sync, long long slot_off) {
  a.world = 1;
  a.rank = 0;
  if (sync) {
    gbh::comm_get(&a.pt, &a.rank, &a.world);
    a.slot_off = slot_off;
    if (a.world > 1) a.epoch = gbh::comm_next_epochs(2);
  }
}

}  // namespace

enum { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2 };

// floats of workspace the BatchNorm entry points need: partials + sums + ready flag
GB_EXPORT long long gb_bn_workspace_floats(int C) { return (long long)C * kSplits * 2 + 2 * C + 8; }

// Forward.  x, y: (N, C, S).  stats: [2C] (mean | invstd), written in training and read
// by backward.  work: gb_bn_workspace_floats(C) floats.  weight / bias: fp32 or null.
// sync != 0: statistics are summed over the ranks of the current communicator through
// the exchange area at slot_off (bytes from the base of the symmetric buffer,
// (2C+1)*world floats).
GB_EXPORT int gb_bn_fwd(int dtype, const void* x, void* y, const float* w, const float* b,
                        float* running_mean, float* running_var, float* stats, float* work, int N,
                        int C, long long S, float eps, float momentum, int training, int relu,
                        int sync, long long slot_off, void* stream) {
  if (C > kMaxC) {
    gbh::set_error("gb_bn_fwd: at most %d channels", kMaxC);
    return gbh::E_TOO_LARGE;
  }
  cudaStream_t s = (cudaStream_t)stream;
  BnArgs a;
  memset(&a, 0, sizeof(a));
  fill_comm(a, sync && training, slot_off);
  a.N = N; a.C = C; a.S = S; a.eps = eps; a.momentum = momentum; a.training = training; a.relu = relu;
  a.part = work; a.sums = work + (long long)C * kSplits * 2; a.stats = stats;
  a.ready = (int*)(work + (long long)C * kSplits * 2 + 2 * C);
  a.ready_val = ++g_ready_counter;
  a.running_mean = running_mean; a.running_var = running_var; a.w = w; a.b = b;
  a.status = gbh::status_ptr();
  const long long total = (long long)N * C * S;
#define GB_BN(T)                                                                                      \
  {                                                                                                   \
    if (training)                                                                                     \
      bn_partial_kernel<T><<<dim3(C, kSplits), 256, 0, s>>>((const T*)x, nullptr, nullptr, nullptr, work, N, C, S, 0); \
    bn_apply_kernel<T><<<grid_for(total), 256, 0, s>>>((const T*)x, (T*)y, a);                        \
  }
  switch (dtype) {
    case DT_BF16: GB_BN(__nv_bfloat16) break;
    case DT_F16: GB_BN(__half) break;
    case DT_F32: GB_BN(float) break;
    default:
      gbh::set_error("gb_bn_fwd: bad dtype %d", dtype);
      return gbh::E_BAD_ARG;
  }
#undef GB_BN
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

// Backward of the training forward.  dgamma / dbeta (fp32, may be null) receive the LOCAL sums.
GB_EXPORT int gb_bn_bwd(int dtype, const void* x, const void* dy, void* dx, const float* w,
                        const float* stats, float* dgamma, float* dbeta, float* work, int N, int C,
                        long long S, int sync, long long slot_off, void* stream) {
  if (C > kMaxC) {
    gbh::set_error("gb_bn_bwd: at most %d channels", kMaxC);
    return gbh::E_TOO_LARGE;
  }
  cudaStream_t s = (cudaStream_t)stream;
  BnArgs a;
  memset(&a, 0, sizeof(a));
  fill_comm(a, sync, slot_off);
  a.N = N; a.C = C; a.S = S; a.training = 1;
  a.part = work; a.sums = work + (long long)C * kSplits * 2; a.stats = const_cast<float*>(stats);
  a.ready = (int*)(work + (long long)C * kSplits * 2 + 2 * C);
  a.ready_val = ++g_ready_counter;
  a.w = w;
  a.status = gbh::status_ptr();
  const long long total = (long long)N * C * S;
#define GB_BN(T)                                                                                      \
  {                                                                                                   \
    bn_partial_kernel<T><<<dim3(C, kSplits), 256, 0, s>>>((const T*)dy, (const T*)x, stats, stats + C, work, N, C, S, 1); \
    bn_bwd_apply_kernel<T><<<grid_for(total), 256, 0, s>>>((const T*)x, (const T*)dy, (T*)dx, dgamma, dbeta, a); \
  }
  switch (dtype) {
    case DT_BF16: GB_BN(__nv_bfloat16) break;
    case DT_F16: GB_BN(__half) break;
    case DT_F32: GB_BN(float) break;
    default:
      gbh::set_error("gb_bn_bwd: bad dtype %d", dtype);
      return gbh::E_BAD_ARG;
  }
#undef GB_BN
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}
