// Bounds-checked debug build.
//
// Compiled with -DGB_BOUNDS_CHECK (python -m gonn_b200.build --debug, which writes a second
// library beside the regular one), the window, embedding, reduction and normalisation kernels
// compare every data-dependent or computed index with the extent of the buffer it addresses
// before they use it.  An index outside the buffer is recorded in the status word (code
// ST_OUT_OF_BOUNDS, detail = the site number given at the call, block index, count) and the access is
// skipped; the kernel carries on and returns normally.  Nothing traps, so the context stays usable
// and the host reads the word with gb_status_read.  This build stands in for a memory checker
// where none can be run; the regular build compiles the checks away.
//
//   if (GB_IN_BOUNDS(src, S, 11)) v = x[base + src];
//   if (GB_IN_EXTENT(blockIdx.x, 0, 12)) part[blockIdx.x * D + c] = v;   // extent slot 0 set by the host
//
// Each translation unit that includes this header keeps its own pointer to the status word
// (no relocatable device code in this library); the host entry points call GB_BOUNDS_BIND()
// before their launches, which stores the pointer once per device.
#pragma once
#include "common.cuh"

#ifdef GB_BOUNDS_CHECK

namespace {
__device__ int* g_bounds_status = nullptr;

__device__ __forceinline__ bool gb_in_bounds(long long i, long long n, int site) {
  if ((unsigned long long)i < (unsigned long long)n) return true;
  gb::set_status(g_bounds_status, gb::ST_OUT_OF_BOUNDS, site);
  return false;
}

// Extents that a kernel's own arguments do not carry (the number of partial rows in a scratch
// buffer, for instance): the host stores them before the launch, in stream order.
__device__ long long g_bounds_extent[4] = {0, 0, 0, 0};

__device__ __forceinline__ bool gb_in_extent(long long i, int slot, int site) {
  return gb_in_bounds(i, g_bounds_extent[slot], site);
}

inline void gb_bounds_extent(int slot, long long value, cudaStream_t stream) {
  cudaMemcpyToSymbolAsync(g_bounds_extent, &value, sizeof(value), slot * sizeof(long long),
                          cudaMemcpyHostToDevice, stream);
}

inline void gb_bounds_bind() {
  static bool bound[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || bound[dev]) return;
  int* p = gbh::status_ptr();
  if (cudaMemcpyToSymbol(g_bounds_status, &p, sizeof(p)) == cudaSuccess) bound[dev] = true;
}
}  // namespace

#define GB_IN_BOUNDS(i, n, site) gb_in_bounds((long long)(i), (long long)(n), (site))
#define GB_IN_EXTENT(i, slot, site) gb_in_extent((long long)(i), (slot), (site))
#define GB_BOUNDS_BIND() gb_bounds_bind()
#define GB_BOUNDS_EXTENT(slot, value, stream) gb_bounds_extent((slot), (long long)(value), (stream))

#else

#define GB_IN_BOUNDS(i, n, site) true
#define GB_IN_EXTENT(i, slot, site) true
#define GB_BOUNDS_BIND() ((void)0)
#define GB_BOUNDS_EXTENT(slot, value, stream) ((void)0)

#endif
