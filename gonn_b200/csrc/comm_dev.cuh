// Device-side building blocks of the peer-memory collectives: the table of peer base
// addresses, epoch-numbered flag slots and the bounded CTA-to-CTA barrier.  Shared by
// comm.cu and by kernels that fuse a small exchange into their own work (batchnorm.cu).
#pragma once
#include "common.cuh"

namespace gbc {
using namespace gb;

constexpr int kMaxWorld = 16;
constexpr int kMaxCtas = 304;
constexpr size_t kFlagBytes = 1 << 20;  // flag area at the start of each symmetric buffer

struct PeerTable {
  void* base[kMaxWorld];  // base address of every rank's symmetric buffer, as mapped here
};

// flag slot: [channel][cta][rank]
__device__ __forceinline__ unsigned int* flag_slot(void* base, int channel, int cta, int rank) {
  return (unsigned int*)base + ((channel * kMaxCtas + cta) * kMaxWorld + rank);
}

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// value + *base (base may be null): see gbh::comm_next_epochs
__device__ __forceinline__ unsigned int dyn_value(unsigned int rel, const unsigned int* base) {
  return base ? rel + __ldcg(base) : rel;
}

// Barrier between CTA `cta` of all ranks.  Thread t < world handles peer t.
// Returns false when the wait ran out of budget.
static __device__ bool cta_barrier(const PeerTable& pt, int rank, int world, int channel, int cta,
                            unsigned int epoch, int* status, int* sm_flag) {
  __syncthreads();  // everything this CTA wrote so far precedes the signal
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(flag_slot(pt.base[threadIdx.x], channel, cta, rank), epoch);
    const unsigned int* mine = flag_slot(pt.base[rank], channel, cta, threadIdx.x);
    const uint64_t t0 = globaltimer_ns();
    unsigned int spins = 0;
    // epochs increase monotonically: ">=" tolerates a peer that is already one call ahead
    while ((int)(ld_acquire_sys(mine) - epoch) < 0) {
      if ((++spins & 0x3F) == 0 && globaltimer_ns() - t0 > kWaitBudgetNs) {
        set_status(status, ST_COMM_TIMEOUT, channel * 1000 + threadIdx.x);
        *sm_flag = 1;
        break;
      }
    }
  }
  __syncthreads();
  return *sm_flag == 0;
}


}  // namespace gbc

// host side (comm.cu): the current communicator
namespace gbh {
void comm_get(gbc::PeerTable* pt, int* rank, int* world);
// Barrier epochs (identical sequence on every rank) and local serial numbers (flags that only
// this rank's kernels compare).  Outside a capture both are absolute and the pointers below are
// null.  Between gb_comm_capture_begin / _end they count from zero and the kernels add the base
// they read from device memory at run time (gbc::dyn_value), so that a CUDA graph can be
// replayed with fresh values: the host writes new bases before every replay.
unsigned int comm_next_epochs(int count);
unsigned int comm_next_serials(int count);
const unsigned int* comm_epoch_base_ptr();
const unsigned int* comm_serial_base_ptr();
}
