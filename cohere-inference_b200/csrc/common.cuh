// Shared device helpers and the host-side error plumbing of the b200dec library (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/b200dec.h"

#define DEVI __device__ __forceinline__

constexpr int D_MODEL = 1024;

// ---- host: error text (thread-local, so concurrent host threads do not share it) ---------------------------------
namespace b200dec_detail {
char* error_buffer();
int fail(int code, const char* fmt, ...);
int check_launch(const char* what);
}  // namespace b200dec_detail

#define B200_REQUIRE(cond, ...)                                                     \
  do {                                                                              \
    if (!(cond)) return b200dec_detail::fail(B200DEC_EINVAL, __VA_ARGS__);          \
  } while (0)

// ---- programmatic dependent launch --------------------------------------------------------------------------------
// Every kernel of the step reads its weights first, then waits for the kernel before it (whose memory is then
// visible), so its prologue overlaps the tail of its predecessor. Both instructions are no-ops in a plain launch.
DEVI void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
DEVI void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Launch with optional cluster size along x and the programmatic-serialization attribute.
template <typename Kern, typename Args>
inline cudaError_t launch_kernel(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster_x,
                                 bool pdl, const Args& args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (cluster_x > 0) {
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = cluster_x;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
  }
  if (pdl) {
    attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, kern, args);
}

// ---- timeline study builds (-DB200DEC_TIMELINE): every launch gets the next slice of a device buffer, 12 slots per
// CTA, and its CTAs store the global nanosecond timer there at their phase boundaries -------------------------------
#ifdef B200DEC_TIMELINE
#define B200DEC_STAMPS 1
namespace b200dec_detail {
long long* timeline_next(int ctas, int kind);  // host side, rowops.cu; nullptr when no buffer is set
}
using b200dec_detail::timeline_next;
DEVI long long stamp_clock() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#else
DEVI long long stamp_clock() { return clock64(); }
#endif

// ---- loads --------------------------------------------------------------------------------------------------------
// Read-once streams (weights, KV cache): no L1 allocation.
DEVI uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
DEVI uint2 ld_stream8(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
DEVI uint32_t ld_stream4(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
// Activations written by the previous kernel: through L2.
DEVI float4 ld_cg_f4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }

DEVI void cp_async16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
DEVI void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// ---- conversions --------------------------------------------------------------------------------------------------
DEVI float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
DEVI float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
DEVI uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
DEVI float clamp_h(float a) { return fminf(fmaxf(a, -65504.f), 65504.f); }
DEVI uint32_t pack_f16(float a, float b) {
  __half2 v = __floats2half2_rn(clamp_h(a), clamp_h(b));
  return *reinterpret_cast<uint32_t*>(&v);
}

DEVI float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
