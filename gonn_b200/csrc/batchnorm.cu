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
// The CTA that finalises is elected at run time: the first CTA to swap this launch's serial
// number into an election word.  It is running by construction, so the CTAs that wait for its
// result never wait for a CTA that has not been dispatched; its own wait for the peers is bounded.
#include "comm_dev.cuh"

using namespace gb;
using namespace gbc;

namespace {

constexpr int kSplits = 32;
constexpr int kMaxC = 2048;

// Four consecutive elements as one 8-byte (16-bit types) or 16-byte (fp32) access.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ void ld(const float* p, float* f) {
    const float4 u = *reinterpret_cast<const float4*>(p);
    f[0] = u.x; f[1] = u.y; f[2] = u.z; f[3] = u.w;
  }
  static __device__ __forceinline__ void st(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ void ld(const __nv_bfloat16* p, float* f) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, const float* f) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]));
  }
};
template <> struct Vec4<__half> {
  static __device__ __forceinline__ void ld(const __half* p, float* f) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    float2 a = unpack_f16(u.x), b = unpack_f16(u.y);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  }
  static __device__ __forceinline__ void st(__half* p, const float* f) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_f16(f[0], f[1]), pack_f16(f[2], f[3]));
  }
};

// Work is handed out by (sample, channel) plane: S contiguous elements that share the
// channel's constants, so the inner loops need no index arithmetic and can be vectorised
// whenever S is a multiple of 4 (plane starts are then 8- / 16-byte aligned).
template <typename T>
__device__ __forceinline__ bool planes_vectorisable(long long S, const void* p0, const void* p1, const void* p2) {
  const uintptr_t m = sizeof(T) * 4 - 1;
  return (S & 3) == 0 && (((uintptr_t)p0 | (uintptr_t)p1 | (uintptr_t)p2) & m) == 0;
}

// partial[c][split][0..1]; mode 0: (x, x^2); mode 1: (dy, dy * xhat).  CTA (c, split):
// the samples of the split, one warp per sample plane at a time.
template <typename T>
__global__ void __launch_bounds__(256)
bn_partial_kernel(const T* __restrict__ a, const T* __restrict__ xin,
                                  const float* __restrict__ mean, const float* __restrict__ invstd,
                                  float* __restrict__ part, int N, int C, long long S, int mode,
                                  const T* __restrict__ yrelu) {
  // yrelu (backward only, may be null): the forward's output after its fused ReLU; the incoming
  // gradient counts as zero wherever that output is zero
  __shared__ float red[32];
  const int c = blockIdx.x, sp = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per = (N + kSplits - 1) / kSplits;
  const int n0 = sp * per, n1 = min(n0 + per, N);
  float s0 = 0.f, s1 = 0.f;
  const float mu = mode ? mean[c] : 0.f, is = mode ? invstd[c] : 0.f;
  const bool vec = planes_vectorisable<T>(S, a, mode ? xin : a, yrelu ? yrelu : a);
  for (int n = n0 + warp; n < n1; n += 8) {
    const long long base = ((long long)n * C + c) * S;
    if (vec) {
      for (long long i = lane * 4; i < S; i += 128) {
        float v[4], xv[4];
        Vec4<T>::ld(a + base + i, v);
        if (mode) Vec4<T>::ld(xin + base + i, xv);
        if (yrelu) {
          float yv[4];
          Vec4<T>::ld(yrelu + base + i, yv);
#pragma unroll
          for (int j = 0; j < 4; j++) v[j] = yv[j] > 0.f ? v[j] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
          s0 += v[j];
          s1 += mode ? v[j] * ((xv[j] - mu) * is) : v[j] * v[j];
        }
      }
    } else {
      for (long long i = lane; i < S; i += 32) {
        float v = (float)a[base + i];
        if (yrelu && !((float)yrelu[base + i] > 0.f)) v = 0.f;
        s0 += v;
        s1 += mode ? v * (((float)xin[base + i] - mu) * is) : v * v;
      }
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
  const unsigned int* epoch_base;   // added to epoch / ready_val at run time when not null
  const unsigned int* serial_base;  // (launches captured in a CUDA graph: see comm_dev.cuh)
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
  int* ready;              // device flag: this launch's serial number once the stats are valid
  int* elect;              // election word: the first CTA to swap the serial number in finalises
  int ready_val;
  int split;               // 1: the statistics were finalised by a separate launch: no flag, no wait;
                           // 2 (one rank): every plane derives them from the partial sums itself, no finalise at all
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
    const unsigned int epoch = dyn_value(a.epoch, a.epoch_base);
    if (!cta_barrier(a.pt, a.rank, a.world, 7, 0, epoch, a.status, sm_flag)) {
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
    cta_barrier(a.pt, a.rank, a.world, 8, 0, epoch + 1, a.status, sm_flag);
  }
  *count_out = count;
  __syncthreads();
}

// One rank: the two sums of channel c from its kSplits partial pairs.  Lane i takes split i and a
// butterfly adds them, so every lane of every warp that does this for the channel gets the same bits
// (a + b == b + a at every level).  Must be called by all 32 lanes.
static_assert(kSplits == 32, "one partial pair per lane");
__device__ __forceinline__ void local_sums(const BnArgs& a, int c, float& s0, float& s1) {
  const int lane = threadIdx.x & 31;
  s0 = __ldcg(a.part + ((long long)c * kSplits + lane) * 2);
  s1 = __ldcg(a.part + ((long long)c * kSplits + lane) * 2 + 1);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s0 += __shfl_xor_sync(0xffffffffu, s0, o);
    s1 += __shfl_xor_sync(0xffffffffu, s1, o);
  }
}

// True in exactly one CTA of the launch: the first to arrive.
__device__ __forceinline__ bool elect_leader(const BnArgs& a, int ready_val) {
  __shared__ int leader;
  if (threadIdx.x == 0) leader = atomicExch(a.elect, ready_val) != ready_val;
  __syncthreads();
  return leader != 0;
}

__device__ __forceinline__ bool wait_ready(const BnArgs& a, int ready_val) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) {
    const uint64_t t0 = globaltimer_ns();
    int ok = 1;
    while (*((volatile int*)a.ready) != ready_val) {
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

// What CTA 0 of the forward does before anybody normalises: combine (and exchange) the
// sums, publish mean / invstd, update the running statistics.
__device__ void bn_fwd_finalise(const BnArgs& a, int* sm_flag, float* s_count) {
  const int C = a.C;
  if (threadIdx.x == 0) *sm_flag = 0;
  __syncthreads();
  float cnt;
  combine_and_exchange(a, a.sums, &cnt, sm_flag);
  if (threadIdx.x == 0) *s_count = cnt;
  __syncthreads();
  const float n = *s_count;
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
}

// The same for the backward: local sums become the parameter gradients, the (exchanged)
// sums divided by the count are left in a.sums.
__device__ void bn_bwd_finalise(const BnArgs& a, float* dgamma, float* dbeta, int* sm_flag, float* s_count) {
  const int C = a.C;
  if (threadIdx.x == 0) *sm_flag = 0;
  __syncthreads();
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
  combine_and_exchange(a, a.sums, &cnt, sm_flag);
  if (threadIdx.x == 0) *s_count = cnt;
  __syncthreads();
  const float n = *s_count;
  for (int c = threadIdx.x; c < 2 * C; c += blockDim.x) a.sums[c] = a.sums[c] / n;
}

// One-CTA launches of the two functions above, used when there is a single rank: the
// normalise kernels then need no device flag (and can be captured in a CUDA graph).
__global__ void __launch_bounds__(256) bn_finalise_kernel(const BnArgs a, float* dgamma, float* dbeta, int backward) {
  __shared__ int sm_flag;
  __shared__ float s_count;
  if (backward) bn_bwd_finalise(a, dgamma, dbeta, &sm_flag, &s_count);
  else bn_fwd_finalise(a, &sm_flag, &s_count);
}

template <typename T>
__global__ void __launch_bounds__(256)
bn_apply_kernel(const T* __restrict__ x, T* __restrict__ y, const BnArgs a) {
  __shared__ int sm_flag;
  __shared__ float s_count;
  const int C = a.C;
  if (a.training && !a.split) {
    const int rv = (int)dyn_value((unsigned int)a.ready_val, a.serial_base);
    if (elect_leader(a, rv)) {
      bn_fwd_finalise(a, &sm_flag, &s_count);
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) atomicExch(a.ready, rv);
    }
    if (!wait_ready(a, rv)) return;
  }
  const float* w = (const float*)a.w;
  const float* b = (const float*)a.b;
  const long long planes = (long long)a.N * C;
  const long long S = a.S;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool vec = planes_vectorisable<T>(S, x, y, x);
  for (long long pl = (long long)blockIdx.x * 8 + warp; pl < planes; pl += (long long)gridDim.x * 8) {
    const int c = (int)(pl % C);
    float mean, is;
    if (a.training && a.split == 2) {
      // single rank: mean and 1/std straight from the partial sums; the planes of the first image
      // publish them for the backward and update the running statistics (one writer per channel)
      float s0, s1;
      local_sums(a, c, s0, s1);
      const float n = (float)a.N * (float)a.S;
      mean = s0 / n;
      float var = s1 / n - mean * mean;
      var = var > 0.f ? var : 0.f;
      is = rsqrtf(var + a.eps);
      if (pl < C && lane == 0) {
        a.stats[c] = mean;
        a.stats[C + c] = is;
        if (a.running_mean) {
          const float unbiased = n > 1.f ? var * n / (n - 1.f) : var;
          a.running_mean[c] = (1.f - a.momentum) * a.running_mean[c] + a.momentum * mean;
          a.running_var[c] = (1.f - a.momentum) * a.running_var[c] + a.momentum * unbiased;
        }
      }
    } else if (a.training) {
      mean = __ldcg(a.stats + c);
      is = __ldcg(a.stats + C + c);
    } else {
      mean = a.running_mean[c];
      is = rsqrtf(a.running_var[c] + a.eps);
    }
    // y = x * scale + shift
    const float scale = w ? is * w[c] : is;
    const float shift = (b ? b[c] : 0.f) - mean * scale;
    const T* xp = x + pl * S;
    T* yp = y + pl * S;
    if (vec) {
      for (long long i = lane * 4; i < S; i += 128) {
        float v[4];
        Vec4<T>::ld(xp + i, v);
#pragma unroll
        for (int j = 0; j < 4; j++) {
          v[j] = fmaf(v[j], scale, shift);
          if (a.relu) v[j] = fmaxf(v[j], 0.f);
        }
        Vec4<T>::st(yp + i, v);
      }
    } else {
      for (long long i = lane; i < S; i += 32) {
        float v = fmaf((float)xp[i], scale, shift);
        if (a.relu) v = fmaxf(v, 0.f);
        yp[i] = (T)v;
      }
    }
  }
}

// dx = w * invstd * (dy - S1/n - xhat * S2/n); dgamma = local S2, dbeta = local S1
template <typename T>
__global__ void __launch_bounds__(256)
bn_bwd_apply_kernel(const T* __restrict__ x, const T* __restrict__ dy, T* __restrict__ dx,
                    float* __restrict__ dgamma, float* __restrict__ dbeta, const BnArgs a,
                    const T* __restrict__ yrelu) {
  __shared__ int sm_flag;
  __shared__ float s_count;
  const int C = a.C;
  if (!a.split) {
    const int rv = (int)dyn_value((unsigned int)a.ready_val, a.serial_base);
    if (elect_leader(a, rv)) {
      bn_bwd_finalise(a, dgamma, dbeta, &sm_flag, &s_count);
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0) atomicExch(a.ready, rv);
    }
    if (!wait_ready(a, rv)) return;
  }
  const float* w = (const float*)a.w;
  const long long planes = (long long)a.N * C;
  const long long S = a.S;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool vec = planes_vectorisable<T>(S, x, dy, dx) && (yrelu == nullptr || planes_vectorisable<T>(S, yrelu, dy, dx));
  for (long long pl = (long long)blockIdx.x * 8 + warp; pl < planes; pl += (long long)gridDim.x * 8) {
    const int c = (int)(pl % C);
    const float mean = a.stats[c], is = a.stats[C + c];
    float m1, m2;
    if (a.split == 2) {
      float s0, s1;
      local_sums(a, c, s0, s1);
      if (pl < C && lane == 0) {
        if (dbeta) dbeta[c] = s0;
        if (dgamma) dgamma[c] = s1;
      }
      const float n = (float)a.N * (float)a.S;
      m1 = s0 / n;
      m2 = s1 / n;
    } else {
      m1 = __ldcg(a.sums + c);
      m2 = __ldcg(a.sums + C + c);
    }
    const float k = w ? is * w[c] : is;
    const T* xp = x + pl * S;
    const T* gp = dy + pl * S;
    T* op = dx + pl * S;
    if (vec) {
      for (long long i = lane * 4; i < S; i += 128) {
        float xv[4], g[4];
        Vec4<T>::ld(xp + i, xv);
        Vec4<T>::ld(gp + i, g);
        if (yrelu) {
          float yv[4];
          Vec4<T>::ld(yrelu + pl * S + i, yv);
#pragma unroll
          for (int j = 0; j < 4; j++) g[j] = yv[j] > 0.f ? g[j] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 4; j++) g[j] = k * (g[j] - m1 - (xv[j] - mean) * is * m2);
        Vec4<T>::st(op + i, g);
      }
    } else {
      for (long long i = lane; i < S; i += 32) {
        float g = (float)gp[i];
        if (yrelu && !((float)yrelu[pl * S + i] > 0.f)) g = 0.f;
        op[i] = (T)(k * (g - m1 - ((float)xp[i] - mean) * is * m2));
      }
    }
  }
}


template <typename T>
__global__ void channel_sum_finish_kernel(const float* __restrict__ part, T* __restrict__ out, int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f;
  for (int sp = 0; sp < kSplits; sp++) s += part[((long long)c * kSplits + sp) * 2];
  out[c] = (T)s;
}

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
  a.epoch_base = gbh::comm_epoch_base_ptr();
  a.serial_base = gbh::comm_serial_base_ptr();
  a.ready_val = (int)gbh::comm_next_serials(1);
}

}  // namespace

enum { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2 };

// floats of workspace the BatchNorm entry points need: partials + sums + ready flag + election
// word; the caller zeroes it once when it allocates it (serial numbers start at 1)
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
  a.elect = a.ready + 1;
  a.running_mean = running_mean; a.running_var = running_var; a.w = w; a.b = b;
  a.split = a.world == 1 ? 2 : 0;
  a.status = gbh::status_ptr();
  const long long total = (long long)N * C * S;
#define GB_BN(T)                                                                                      \
  {                                                                                                   \
    if (training)                                                                                     \
      bn_partial_kernel<T><<<dim3(C, kSplits), 256, 0, s>>>((const T*)x, nullptr, nullptr, nullptr, work, N, C, S, 0, nullptr); \
    if (training && a.split == 1) bn_finalise_kernel<<<1, 256, 0, s>>>(a, nullptr, nullptr, 0);       \
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

// out[c] = sum over n and s of x[n][c][s] (a convolution's bias gradient), in the tensor's dtype.
// work: gb_bn_workspace_floats(C) floats.  Two launches: the per-channel partial sums of the
// BatchNorm forward, then one thread per channel adds the kSplits partials in order.
GB_EXPORT int gb_channel_sum(int dtype, const void* x, void* out, float* work, int N, int C, long long S,
                             void* stream) {
  if (C > kMaxC) {
    gbh::set_error("gb_channel_sum: at most %d channels", kMaxC);
    return gbh::E_TOO_LARGE;
  }
  if (N <= 0 || C <= 0 || S <= 0) return gbh::E_OK;
  cudaStream_t s = (cudaStream_t)stream;
#define GB_CS(T)                                                                                              \
  {                                                                                                           \
    bn_partial_kernel<T><<<dim3(C, kSplits), 256, 0, s>>>((const T*)x, nullptr, nullptr, nullptr, work, N, C, S, 0, \
                                                          nullptr);                                           \
    channel_sum_finish_kernel<T><<<(C + 127) / 128, 128, 0, s>>>(work, (T*)out, C);                           \
  }
  switch (dtype) {
    case DT_BF16: GB_CS(__nv_bfloat16) break;
    case DT_F16: GB_CS(__half) break;
    case DT_F32: GB_CS(float) break;
    default:
      gbh::set_error("gb_channel_sum: bad dtype %d", dtype);
      return gbh::E_BAD_ARG;
  }
#undef GB_CS
  GB_CUDA_OK(cudaGetLastError());
  return gbh::E_OK;
}

// Backward of the training forward.  dgamma / dbeta (fp32, may be null) receive the LOCAL sums.
// yrelu (may be null): the forward's output when it had the ReLU fused in; the gradient is then
// masked by (yrelu > 0) inside both kernels instead of by separate elementwise launches.
GB_EXPORT int gb_bn_bwd(int dtype, const void* x, const void* dy, void* dx, const float* w,
                        const float* stats, float* dgamma, float* dbeta, float* work, int N, int C,
                        long long S, int sync, long long slot_off, const void* yrelu, void* stream) {
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
  a.elect = a.ready + 1;
  a.w = w;
  a.split = a.world == 1 ? 2 : 0;
  a.status = gbh::status_ptr();
  const long long total = (long long)N * C * S;
#define GB_BN(T)                                                                                      \
  {                                                                                                   \
    bn_partial_kernel<T><<<dim3(C, kSplits), 256, 0, s>>>((const T*)dy, (const T*)x, stats, stats + C, work, N, C, S, 1, (const T*)yrelu); \
    if (a.split == 1) bn_finalise_kernel<<<1, 256, 0, s>>>(a, dgamma, dbeta, 1);                      \
    bn_bwd_apply_kernel<T><<<grid_for(total), 256, 0, s>>>((const T*)x, (const T*)dy, (T*)dx, dgamma, dbeta, a, (const T*)yrelu); \
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
