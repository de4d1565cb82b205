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

// the weight kinds of the tcgen05 kernels (linear_umma.cu, head_umma.cu)
inline bool is_umma_kind(int kind) {
  return kind == B200DEC_W_INT8_UMMA || kind == B200DEC_W_F16_UMMA || kind == B200DEC_W_INT8_24_UMMA;
}
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

// ---- thread-block clusters -----------------------------------------------------------------------------------------
// A CTA may touch the shared memory of another CTA of its cluster only once that CTA has started. Every clustered
// kernel therefore arrives at the cluster barrier as its first instruction and completes that phase (the wait) just
// before its first remote store; in between lie the weight prefetch and the wait for the previous kernel, so the
// pair costs nothing on the critical path. Each thread that arrives must wait before it arrives again (cluster.sync()).
DEVI void cluster_arrive_entry() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
DEVI void cluster_wait_entry() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }

// ---- exchange of partial results inside a cluster without a barrier -------------------------------------------------
// Every store into a peer's shared memory (st.async) also counts its bytes on an mbarrier of that peer; a CTA that
// knows how many bytes it is owed waits on its own mbarrier only (bounded), instead of a barrier across the cluster that
// first has to see every CTA's stores acknowledged. A CTA leaves once it holds everything it is owed, so nobody writes
// into a CTA that has gone. The mbarrier is initialised before the entry arrive (release) above, and peers complete
// that phase (acquire) before their first store, so it is never touched uninitialised.
DEVI uint32_t smem_addr_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
DEVI uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {  // the same shared-memory offset in CTA `rank`
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
DEVI void st_async_f32(uint32_t remote_addr, float v, uint32_t remote_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(remote_addr),
               "r"(__float_as_uint(v)), "r"(remote_bar)
               : "memory");
}
DEVI void st_async_f32x2(uint32_t remote_addr, float2 v, uint32_t remote_bar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v2.b32 [%0], {%1, %2}, [%3];" ::"r"(remote_addr),
               "r"(__float_as_uint(v.x)), "r"(__float_as_uint(v.y)), "r"(remote_bar)
               : "memory");
}
DEVI void xbar_init(uint64_t* bar) {  // one arrival: the owner's expect_tx
  asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr_u32(bar)));
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
DEVI void xbar_expect(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr_u32(bar)), "r"(bytes) : "memory");
}
DEVI bool xbar_wait(uint64_t* bar, uint32_t limit) {  // phase 0; false when the limit ran out
  const uint32_t addr = smem_addr_u32(bar);
  for (uint32_t i = 0; i < limit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(addr), "r"(0)
        : "memory");
    if (done) return true;
  }
  return false;
}

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
DEVI void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
DEVI void cp_async_wait_group() {  // until at most N of this thread's committed groups are still in flight
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---- prefetch of an attention launch's keys and values into L2 -----------------------------------------------------
// The step alternates between projections (bound by latency, HBM nearly idle) and attention (bound by HBM). A
// projection that runs between two attention launches can therefore start the next launch's cache stream early: its
// threads issue L2 prefetches over runs of keys and values and go on; nothing waits for them. The rows come from the
// step's row schedule (b200dec_row_schedule), whose fourth word is the number of keys of the row to prefetch (the launch's total is capped by the plan's budget so that it stays inside L2).
struct KvPrefetch {
  const int4* sched;  // (rows, 4) {row, slot, length, keys to prefetch}; null: nothing to do
  const char* k;      // caches (slots + 1, H, cap, vec_bytes)
  const char* v;
  int rows, heads, cap, vec_bytes, slots;  // slots: the last valid slot index (the dummy)
};
DEVI void prefetch_l2_line(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
// Called by every thread of every CTA of a grid of `nctas` CTAs (this one's index `cta`, `nthreads` threads each): the
// grid's CTAs share out the (row, head, key | value) runs, a CTA's threads the 128-byte lines of a run (slots and key
// counts are clamped into the caches first).
DEVI void kv_prefetch_issue(const KvPrefetch& f, int cta, int nctas, int tid, int nthreads) {
  const int ops = f.rows * f.heads * 2;
  for (int o = cta; o < ops; o += nctas) {
    const int i = o / (2 * f.heads), rem = o % (2 * f.heads), h = rem >> 1;
    const int4 e = __ldcg(f.sched + i);
    const int keys = e.w < f.cap ? e.w : f.cap;
    if (keys <= 0 || e.y < 0 || e.y > f.slots) continue;
    const char* src = ((rem & 1) ? f.v : f.k) + ((size_t)e.y * f.heads + h) * f.cap * f.vec_bytes;
    const int bytes = keys * f.vec_bytes;
    for (int off = tid * 128; off < bytes; off += nthreads * 128) prefetch_l2_line(src + off);
  }
}

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
