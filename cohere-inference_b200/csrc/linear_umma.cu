// The layer projections on the fifth-generation tensor cores, for dense int8 weights:
// out(rows, N) = act(a' W^T * scale + bias) [+ out], a' = the fp16 rows a or LayerNorm of the rows behind a ready
// fp16 operand; rows <= 128, K = 1024 (split 4 or 8 ways) or 4096 (8 ways; above 64 rows dealt as two clusters of 64 rows per tile), N a multiple of 128.
//
// Same decomposition as the mma.sync kernel of linear_kernel.cuh with 128 channels per CTA and K split over a
// cluster, but the multiply is 8-32 `tcgen05.mma` (M = 128 channels, N = 64 or 128 rows, K = 16) into tensor memory
// instead of 64-256 `mma.sync` per warp:
//   * weights: the CTA's four 8 KB blocks (b200dec_tile_int8_umma layout) go to registers before the dependency wait,
//     are widened to fp16 (exact) and written as K-major 128-byte-swizzled tiles;
//   * activations: the ready operand of the LayerNorm (row * gamma as fp16, see b200dec_ln_link) is copied with
//     cp.async straight into swizzled tiles; the rows' statistics are added up by the cluster from the producer's
//     partial sums, as in the mma.sync kernel;
//   * D(128 x rows) comes back with tcgen05.ld (thread = channel), each warp pushes its 32 channels to the CTA of the
//     cluster that owns them (128-byte rows through distributed shared memory), one cluster barrier, then the same
//     epilogue: y = rstd * (acc * scale - mean * g) + ln_bias + bias (or acc * scale + bias), activation, fp16 or fp32
//     store or add into the residual stream, and for a projection that updates the stream the next LayerNorm's
//     operand and partial sums (b200dec_ln_link).
// fp16 weights (B200DEC_W_F16_UMMA, template flag W16) are stored as the images of those swizzled tiles
// (b200dec_tile_f16_umma): one lane copies the CTA's blocks from HBM into the A tiles with `cp.async.bulk` onto an
// mbarrier before the dependency wait, no thread touches a weight, and the MMA lane waits for that barrier.
// 2:4 int8 weights (B200DEC_W_INT8_24_UMMA, b200dec_tile_24_umma): a thread's 32 k of a block are 16 kept bytes and one
// selector word of compress_24's format; it expands them to the dense fp16 tile (a byte permute per group of four from
// a 32-entry control table, then the same exact widening) and the multiply is the dense one.
// The waits for the copies and the MMAs are bounded (B200DEC_ST_TIMEOUT); tensor memory is released on every path.
#include <cooperative_groups.h>

#include "common.cuh"

using namespace b200dec_detail;
namespace cg = cooperative_groups;

namespace {

constexpr int UM = 128;             // channels per CTA (MMA M)
constexpr int KB = 64;              // k per block: one 128-byte row of fp16
constexpr int RAW_BYTES = UM * KB;  // 8 KB of uint8 per block
constexpr int A_BYTES = UM * KB * 2;
constexpr int NTHREADS = 256;
constexpr uint32_t WAIT_LIMIT = 1u << 22;

struct UArgs {
  const uint8_t* w;
  const uint32_t* meta;  // 2:4: the selector words
  const float* scale;
  const float* bias;     // may be null
  const __half* xg;      // (rows, lda) fp16: the operand rows (with a LayerNorm: row * gamma)
  const float* stats;    // LayerNorm: (rows, stats_slots, 2) partial sums of the rows
  const float* ln_g;
  const float* ln_bias;
  void* out;
  // a projection that updates the residual stream: the next LayerNorm's operand and partial sums (or null)
  const float* next_gamma;
  __half* out16;
  float* stats_out;
  int* status;
  float ln_eps;
  int lda, ldo, rows, N, K, out_kind, act, stats_slots;
  uint32_t wait_limit;  // polls before the wait for the MMAs gives up
  int withhold;         // tests only: the commit is left out, so that wait runs out
  int deal;             // host side only: more than 64 rows go as clusters of 64 rows over grid.z, not one 128-row tile
};

// MB: row capacity (MMA N); KSPLIT: CTAs per cluster; NKB: 64-k blocks per CTA
template <int MB, int KSPLIT, int NKB>
struct USmem {
  static constexpr int CPR = UM / KSPLIT;       // channels finished by each CTA
  static constexpr int XB_BYTES = MB * KB * 2;  // one k-block of the activations
  static constexpr int OFF_A = 0, OFF_X = NKB * A_BYTES, OFF_RECV = OFF_X + NKB * XB_BYTES,
                       OFF_STATS = OFF_RECV + KSPLIT * MB * CPR * 4, USED = OFF_STATS + MB * 8;
  static constexpr int BYTES = USED + 1024;  // slack to align the base to a swizzle atom
};

DEVI uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
DEVI void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
DEVI void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
DEVI void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
DEVI bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit) {  // bounded; false when the limit ran out
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < limit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
// K-major tile with the 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart
DEVI uint64_t umma_desc(uint32_t saddr) {
  uint64_t d = (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
template <int N>
DEVI void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
  // fp16 x fp16 -> fp32, both operands K-major, M = 128
  constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(UM >> 4) << 24);
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}
DEVI void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
DEVI void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// 16 values of uint8 = q + 128 -> 16 exact fp16 q
DEVI void widen16(const uint4& r, uint4& lo, uint4& hi) {
  const uint32_t in[4] = {r.x, r.y, r.z, r.w};
  uint32_t out[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t a = __byte_perm(in[i], 0x64646464u, 0x4140), b = __byte_perm(in[i], 0x64646464u, 0x4342);
    const __half2 off = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));
    const __half2 ha = __hsub2(*reinterpret_cast<const __half2*>(&a), off);
    const __half2 hb = __hsub2(*reinterpret_cast<const __half2*>(&b), off);
    out[2 * i] = *reinterpret_cast<const uint32_t*>(&ha), out[2 * i + 1] = *reinterpret_cast<const uint32_t*>(&hb);
  }
  lo = make_uint4(out[0], out[1], out[2], out[3]), hi = make_uint4(out[4], out[5], out[6], out[7]);
}
// 4 offset-binary bytes (q + 128, k .. k + 3) -> half2(q0, q1), half2(q2, q3), exact
DEVI void widen_u8x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t a = __byte_perm(w, 0x64646464u, 0x4140), b = __byte_perm(w, 0x64646464u, 0x4342);
  const __half2 off = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));
  const __half2 ha = __hsub2(*reinterpret_cast<const __half2*>(&a), off);
  const __half2 hb = __hsub2(*reinterpret_cast<const __half2*>(&b), off);
  lo = *reinterpret_cast<const uint32_t*>(&ha), hi = *reinterpret_cast<const uint32_t*>(&hb);
}
DEVI float act_fn(float v, int act) {
  if (act == B200DEC_ACT_RELU) return fmaxf(v, 0.f);
  if (act == B200DEC_ACT_GELU) return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
  return v;
}
// 32 consecutive columns of this warp's 32 tensor-memory lanes
DEVI void tmem_ld32(uint32_t taddr, uint32_t (&d)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]), "=r"(d[8]),
        "=r"(d[9]), "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15]), "=r"(d[16]),
        "=r"(d[17]), "=r"(d[18]), "=r"(d[19]), "=r"(d[20]), "=r"(d[21]), "=r"(d[22]), "=r"(d[23]), "=r"(d[24]),
        "=r"(d[25]), "=r"(d[26]), "=r"(d[27]), "=r"(d[28]), "=r"(d[29]), "=r"(d[30]), "=r"(d[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// WK: how the weights come: 0 dense int8 blocks, 1 fp16 tile images (bulk copy), 2 2:4 int8 (kept values + selectors)
template <int MB, int KSPLIT, int NKB, bool LN, int WK>
__global__ void __launch_bounds__(NTHREADS, 1) linear_umma_kernel(const UArgs p_in) {
  constexpr bool W16 = WK == 1, W24 = WK == 2;
  // rows dealt over grid.z: this cluster takes rows [MB z, MB z + MB) of the call (every pointer indexed by row moves)
  UArgs p = p_in;
  if (blockIdx.z) {
    const int row0 = blockIdx.z * MB;
    p.rows = min(MB, p.rows - row0);
    p.xg += (size_t)row0 * p.lda;
    p.out = (char*)p.out + (size_t)row0 * p.ldo * (p.out_kind == B200DEC_OUT_F16 ? 2 : 4);
    if (p.stats) p.stats += (size_t)row0 * p.stats_slots * 2;
    if (p.out16) p.out16 += (size_t)row0 * p.ldo;
    if (p.stats_out) p.stats_out += (size_t)row0 * (gridDim.y * KSPLIT) * 2;
  } else if (gridDim.z > 1) {
    p.rows = min(MB, p.rows);
  }
  using S = USmem<MB, KSPLIT, NKB>;
  constexpr int CPR = S::CPR, GPR = CPR / 4, KSLICE = NKB * KB;
  extern __shared__ unsigned char dyn_smem[];
  unsigned char* smem = dyn_smem + ((1024 - (smem_u32(dyn_smem) & 1023)) & 1023);
  unsigned char* as = smem + S::OFF_A;
  unsigned char* xs = smem + S::OFF_X;
  float* recv = reinterpret_cast<float*>(smem + S::OFF_RECV);  // [KSPLIT][MB][CPR]
  float2* stats = reinterpret_cast<float2*>(smem + S::OFF_STATS);
  __shared__ __align__(8) uint64_t d_full, w_full;
  __shared__ uint32_t tmem_base;
  __shared__ uint32_t lut[32];

  cluster_arrive_entry();  // completed by cluster_wait_entry() before this CTA's first remote store
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = blockIdx.x, tile = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ch = (warp & 3) * 32 + lane;  // this thread's channel of the tile = its tensor-memory lane
  const int hf = warp >> 2;               // its half: 16-k pieces 2 hf, 2 hf + 1 of a block; rows hf * MB / 2 ..

  // ---- prologue: the CTA's weight blocks into registers (independent of the previous kernel) ----------------------
  uint4 wr[W16 ? 1 : NKB][W24 ? 1 : 2];
  uint32_t mr[W24 ? NKB : 1];
  if constexpr (WK == 0) {
    const uint8_t* wsrc = p.w + ((size_t)tile * (p.K / KB) + rank * NKB) * RAW_BYTES + ch * 16;
#pragma unroll
    for (int b = 0; b < NKB; ++b)
#pragma unroll
      for (int j = 0; j < 2; ++j) wr[b][j] = ld_stream16(wsrc + (size_t)b * RAW_BYTES + (2 * hf + j) * 2048);
  }
  if constexpr (W24) {  // this thread's 32 k of a block: 16 kept bytes and the eight selectors of its groups of four
    const size_t blk0 = (size_t)tile * (p.K / KB) + rank * NKB;
    const uint8_t* wsrc = p.w + blk0 * (RAW_BYTES / 2) + hf * 2048 + ch * 16;
    const uint32_t* msrc = p.meta + blk0 * 256 + hf * 128 + ch;
#pragma unroll
    for (int b = 0; b < NKB; ++b) {
      wr[b][0] = ld_stream16(wsrc + (size_t)b * (RAW_BYTES / 2));
      mr[b] = ld_stream4(msrc + (size_t)b * 256);
    }
    // byte-permute controls: dense byte q of a group takes kept byte 0/1 (even group of the register) or 2/3 (odd) when
    // q is the first / second kept position, else the zero byte (index 4 = 0x80 in offset binary)
    if (tid < 32) {
      const int i0 = tid & 3, i1 = (tid >> 2) & 3, odd = tid >> 4;
      uint32_t ctl = 0;
      for (int q = 0; q < 4; ++q) {
        uint32_t sel = 4;
        if (q == i1) sel = odd ? 3 : 1;
        if (q == i0) sel = odd ? 2 : 0;
        ctl |= sel << (4 * q);
      }
      lut[tid] = ctl;
    }
  }
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&d_full)));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&w_full)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if constexpr (W16) {  // the CTA's blocks are the tiles' images: HBM -> A tiles, no thread in between
      const uint8_t* wsrc = p.w + ((size_t)tile * (p.K / KB) + rank * NKB) * A_BYTES;
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&w_full)), "r"(NKB * A_BYTES)
                   : "memory");
#pragma unroll
      for (int b = 0; b < NKB; ++b) bulk_load(as + b * A_BYTES, wsrc + (size_t)b * A_BYTES, A_BYTES, &w_full);
    }
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base)), "n"(MB)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // ---- widen the weights into the A tiles: they depend on nothing the previous kernel writes, so this happens in
  // front of the dependency wait, under the previous kernel's tail (the tiles are this CTA's own shared memory)
  if constexpr (W24) {
    __syncthreads();  // the control table
#pragma unroll
    for (int b = 0; b < NKB; ++b) {
      unsigned char* row = as + b * A_BYTES + (ch >> 3) * 1024 + (ch & 7) * 128;
      const uint32_t kw[4] = {wr[b][0].x ^ 0x80808080u, wr[b][0].y ^ 0x80808080u, wr[b][0].z ^ 0x80808080u,
                              wr[b][0].w ^ 0x80808080u};
#pragma unroll
      for (int c = 0; c < 4; ++c) {  // register c = groups 2 c, 2 c + 1 = k 8 c .. 8 c + 7 of the 32 = one 16-byte chunk
        uint32_t o[4];
        widen_u8x4(__byte_perm(kw[c], 0x80808080u, lut[(mr[b] >> (8 * c)) & 15u]), o[0], o[1]);
        widen_u8x4(__byte_perm(kw[c], 0x80808080u, lut[((mr[b] >> (8 * c + 4)) & 15u) | 16u]), o[2], o[3]);
        *reinterpret_cast<uint4*>(row + (((4 * hf + c) ^ (ch & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
  if constexpr (WK == 0) {
#pragma unroll
    for (int b = 0; b < NKB; ++b) {
      unsigned char* row = as + b * A_BYTES + (ch >> 3) * 1024 + (ch & 7) * 128;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int pj = 2 * hf + j;  // k = 16 pj .. 16 pj + 15 of the block: chunks 2 pj and 2 pj + 1 of the row
        uint4 lo, hi;
        widen16(wr[b][j], lo, hi);
        *reinterpret_cast<uint4*>(row + (((2 * pj) ^ (ch & 7)) << 4)) = lo;
        *reinterpret_cast<uint4*>(row + (((2 * pj + 1) ^ (ch & 7)) << 4)) = hi;
      }
    }
  }
  pdl_wait();
  pdl_trigger();  // at once: the dependent's CTAs need ~2 us to start and fetch their weights, more than is left of this one

  // ---- stage this K slice of the operand into swizzled tiles; the cluster adds up the rows' statistics -------------
  const int k0 = rank * KSLICE;
  constexpr int CH = KSLICE / 8;  // 16-byte chunks per row
  for (int i = tid; i < MB * CH; i += NTHREADS) {
    const int r = i / CH, c = i % CH, kb = c >> 3, chunk = c & 7;
    unsigned char* dst = xs + kb * S::XB_BYTES + (r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4);
    if (r < p.rows) cp_async16(dst, p.xg + (size_t)r * p.lda + k0 + c * 8);
    else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
  }
  if constexpr (LN) {
    constexpr int RPW = (MB + KSPLIT * 8 - 1) / (KSPLIT * 8);  // rows per warp, all their loads issued at once
    float2 v[RPW][4];
#pragma unroll
    for (int j = 0; j < RPW; ++j) {
      const int r = rank + KSPLIT * (warp + 8 * j);
      const float2* part = reinterpret_cast<const float2*>(p.stats) + (size_t)r * p.stats_slots;
#pragma unroll
      for (int i = 0; i < 4; ++i)
        v[j][i] = (r < p.rows && lane + 32 * i < p.stats_slots) ? __ldcg(part + lane + 32 * i) : make_float2(0.f, 0.f);
    }
    cluster_wait_entry();
#pragma unroll
    for (int j = 0; j < RPW; ++j) {
      const int r = rank + KSPLIT * (warp + 8 * j);
      float s1 = (v[j][0].x + v[j][1].x) + (v[j][2].x + v[j][3].x), s2 = (v[j][0].y + v[j][1].y) + (v[j][2].y + v[j][3].y);
      s1 = warp_sum(s1), s2 = warp_sum(s2);
      if (r < p.rows && lane < KSPLIT) cluster.map_shared_rank(stats, lane)[r] = make_float2(s1, s2);
    }
  }
  cp_async_wait_all();
  fence_async_shared();  // the MMA reads both operands through the async proxy
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = tmem_base;

  // ---- multiply: one lane, 4 instructions per block, completion through an mbarrier ---------------------------------
  bool w_ok = true;
  if (tid == 0) {
    if constexpr (W16) {
      w_ok = mbar_wait(&w_full, 0, p.wait_limit);  // the weight tiles have landed (async proxy: no fence needed)
      if (!w_ok) atomicOr(p.status, B200DEC_ST_TIMEOUT);
    }
    // the descriptors of block 0; a k-step of 16 advances a tile's start by 32 bytes = 2 units of its address field, a
    // block by the tile's size (the tiles are 1 KB aligned and lie below 256 KB: no carry out of the field)
    const uint64_t da = umma_desc(smem_u32(as)), db = umma_desc(smem_u32(xs));
#pragma unroll
    for (int b = 0; b < NKB; ++b) {
#pragma unroll
      for (int k = 0; k < KB / 16; ++k)
        umma_f16<MB>(tmem_d, da + (uint64_t)(b * (A_BYTES >> 4) + 2 * k), db + (uint64_t)(b * (S::XB_BYTES >> 4) + 2 * k),
                     (b | k) != 0);
    }
    if (!p.withhold) umma_commit(&d_full);
  }
  const bool got = mbar_wait(&d_full, 0, p.wait_limit);
  if (!got && lane == 0) atomicOr(p.status, B200DEC_ST_TIMEOUT);
  tc_fence_after();

  // ---- partial tile -> the CTAs that own its channels (CPR consecutive channels each) ---------------------------------
  if constexpr (!LN) cluster_wait_entry();  // with a LayerNorm the statistics were the first remote stores
  {
    float* dst = cluster.map_shared_rank(recv, ch / CPR) + (size_t)rank * MB * CPR + ch % CPR;
#pragma unroll
    for (int c0 = 0; c0 < MB / 2; c0 += 32) {
      uint32_t d[32];
      tmem_ld32(tmem_d + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(hf * (MB / 2) + c0), d);
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int r = hf * (MB / 2) + c0 + i;
        if (r < p.rows) dst[r * CPR] = __uint_as_float(d[i]);
      }
    }
  }
  // the per-channel vectors of the epilogue (and the residual, for one item per thread), fetched before the barrier
  const int items = p.rows * GPR;
  const int n_mine = tile * UM + rank * CPR + (tid % GPR) * 4;
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f), one4 = make_float4(1.f, 1.f, 1.f, 1.f);
  const float4 sc = p.scale ? __ldg(reinterpret_cast<const float4*>(p.scale + n_mine)) : one4;
  const float4 gg = LN ? __ldg(reinterpret_cast<const float4*>(p.ln_g + n_mine)) : zero4;
  const float4 lb = LN ? __ldg(reinterpret_cast<const float4*>(p.ln_bias + n_mine)) : zero4;
  const float4 bb = p.bias ? __ldg(reinterpret_cast<const float4*>(p.bias + n_mine)) : zero4;
  const float4 gn = p.out16 ? __ldg(reinterpret_cast<const float4*>(p.next_gamma + n_mine)) : one4;
  const bool add = p.out_kind == B200DEC_OUT_F32_ADD;
  float4 resid = zero4;
  if (add && tid < items)
    resid = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.out) + (size_t)(tid / GPR) * p.ldo + n_mine));
  tc_fence_before();
  cluster.sync();  // all partials and statistics have landed; nobody touches remote shared memory after this

  const int padded = (items + 31) & ~31;
  for (int it = tid; it < padded; it += NTHREADS) {  // NTHREADS % GPR == 0: a thread keeps its four channels
    const bool live = it < items;
    const int r = live ? it / GPR : 0, c4 = it % GPR;
    const int n = tile * UM + rank * CPR + c4 * 4;
    float4 s = zero4;
    if (live) {
#pragma unroll
      for (int q = 0; q < KSPLIT; ++q) {  // fixed rank order
        const float4 v = *reinterpret_cast<const float4*>(recv + (q * MB + r) * CPR + c4 * 4);
        s.x += v.x, s.y += v.y, s.z += v.z, s.w += v.w;
      }
      s.x *= sc.x, s.y *= sc.y, s.z *= sc.z, s.w *= sc.w;
      if constexpr (LN) {
        const float2 st = stats[r];
        const float mean = st.x * (1.f / D_MODEL);
        const float rstd = rsqrtf(fmaxf(st.y * (1.f / D_MODEL) - mean * mean, 0.f) + p.ln_eps);
        s.x = rstd * (s.x - mean * gg.x) + lb.x, s.y = rstd * (s.y - mean * gg.y) + lb.y;
        s.z = rstd * (s.z - mean * gg.z) + lb.z, s.w = rstd * (s.w - mean * gg.w) + lb.w;
      }
      s.x += bb.x, s.y += bb.y, s.z += bb.z, s.w += bb.w;
      s.x = act_fn(s.x, p.act), s.y = act_fn(s.y, p.act), s.z = act_fn(s.z, p.act), s.w = act_fn(s.w, p.act);
      if (p.out_kind == B200DEC_OUT_F16) {
        *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(p.out) + (size_t)r * p.ldo + n) =
            make_uint2(pack_f16(s.x, s.y), pack_f16(s.z, s.w));
      } else {
        float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + (size_t)r * p.ldo + n);
        if (add) {
          const float4 x = it == tid ? resid : __ldcg(o);
          s.x += x.x, s.y += x.y, s.z += x.z, s.w += x.w;
          if (p.out16)
            *reinterpret_cast<uint2*>(p.out16 + (size_t)r * p.ldo + n) =
                make_uint2(pack_f16(s.x * gn.x, s.y * gn.y), pack_f16(s.z * gn.z, s.w * gn.w));
        }
        *o = s;
      }
    }
    if (p.stats_out) {  // warp-uniform; the row's GPR consecutive lanes add up their channels, one of them publishes
      float p1 = live ? (s.x + s.y) + (s.z + s.w) : 0.f;
      float p2 = live ? (s.x * s.x + s.y * s.y) + (s.z * s.z + s.w * s.w) : 0.f;
#pragma unroll
      for (int o = 1; o < GPR; o <<= 1) {
        p1 += __shfl_xor_sync(0xffffffffu, p1, o);
        p2 += __shfl_xor_sync(0xffffffffu, p2, o);
      }
      if (live && c4 == 0)
        reinterpret_cast<float2*>(p.stats_out)[(size_t)r * (gridDim.y * KSPLIT) + tile * KSPLIT + rank] = make_float2(p1, p2);
    }
  }
  // ---- release the tensor memory ----------------------------------------------------------------------------------------
  if constexpr (W16) {  // copies that had not landed in time get a second bounded chance before the tiles are given away
    if (tid == 0 && !w_ok) mbar_wait(&w_full, 0, p.wait_limit);
  }
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "n"(MB) : "memory");
  }
}

// kept (n, k / 2) int8 and words (n, k / 32) of compress_24 -> blocks [n / 128][k / 64]: 4 KB of kept bytes
// [half of the block's k][channel][16 bytes] and 256 selector words [half][channel] (a half = 32 k = one word of the row)
__global__ void tile_24_umma_kernel(const int8_t* __restrict__ kept, const uint32_t* __restrict__ words, int n, int k,
                                    uint8_t* __restrict__ out, uint32_t* __restrict__ meta) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // one kept byte each
  if (i >= (size_t)n * (k / 2)) return;
  const int e = i & 15, t = (i >> 4) & 127, hf = (i >> 11) & 1;
  const size_t blk = i >> 12;
  const int nkb = k / KB, kb = (int)(blk % nkb), mt = (int)(blk / nkb);
  const size_t row = (size_t)mt * UM + t;
  out[i] = (uint8_t)kept[row * (k / 2) + kb * 32 + hf * 16 + e];
  if (e == 0) meta[blk * 256 + hf * 128 + t] = words[row * (k / 32) + kb * 2 + hf];
}

template <int MB, int KSPLIT, int NKB, bool LN, int WK>
int launch_umma(const UArgs& a, int pdl, cudaStream_t stream) {
  using S = USmem<MB, KSPLIT, NKB>;
  if constexpr (S::BYTES > 227 * 1024 - 512) {
    return fail(B200DEC_EINVAL, "linear_umma: %d rows of K / %d do not fit shared memory", MB, KSPLIT);
  } else {
    auto kern = linear_umma_kernel<MB, KSPLIT, NKB, LN, WK>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::BYTES);
    if (e != cudaSuccess) return fail(B200DEC_ECUDA, "linear_umma: smem attribute: %s", cudaGetErrorString(e));
    e = launch_kernel(kern, dim3(KSPLIT, a.N / UM, (a.rows + MB - 1) / MB), dim3(NTHREADS), S::BYTES, stream, KSPLIT, pdl, a);
    if (e != cudaSuccess) return fail(B200DEC_ECUDA, "linear_umma launch: %s", cudaGetErrorString(e));
    return 0;
  }
}

template <int KSPLIT, int NKB, int WK>
int launch_rows_wk(const UArgs& a, bool ln, int pdl, cudaStream_t s) {
  // 64-row tiles: up to 64 rows, and above that where the rows are dealt over two clusters per tile (a.deal)
  if (a.rows <= 64 || a.deal)
    return ln ? launch_umma<64, KSPLIT, NKB, true, WK>(a, pdl, s) : launch_umma<64, KSPLIT, NKB, false, WK>(a, pdl, s);
  return ln ? launch_umma<128, KSPLIT, NKB, true, WK>(a, pdl, s) : launch_umma<128, KSPLIT, NKB, false, WK>(a, pdl, s);
}
template <int KSPLIT, int NKB>
int launch_rows(const UArgs& a, int wk, bool ln, int pdl, cudaStream_t s) {
  return wk == 1 ? launch_rows_wk<KSPLIT, NKB, 1>(a, ln, pdl, s)
       : wk == 2 ? launch_rows_wk<KSPLIT, NKB, 2>(a, ln, pdl, s) : launch_rows_wk<KSPLIT, NKB, 0>(a, ln, pdl, s);
}

}  // namespace

namespace b200dec_detail {

// A projection whose weight is of kind B200DEC_W_INT8_UMMA, B200DEC_W_F16_UMMA or B200DEC_W_INT8_24_UMMA. a: fp16 rows; with ln they are the LayerNorm's ready
// operand and link->stats_in its partial sums (b200dec_ln_link). w->ksplit: CTAs per cluster (K = 1024: 4 or 8;
// K = 4096: 8).
int linear_umma_impl(const b200dec_weight* w, const void* a, int a_kind, const b200dec_norm* ln, int lda, int rows,
                     void* out, int out_kind, int ldo, int act, const b200dec_ln_link* link, int32_t* status, int pdl,
                     void* stream) {
  B200_REQUIRE(w && w->w && a && out && status, "linear_umma: null pointer");
  const bool w16 = w->kind == B200DEC_W_F16_UMMA, w24 = w->kind == B200DEC_W_INT8_24_UMMA;
  B200_REQUIRE(w16 == (w->scale == nullptr) && ((uintptr_t)w->w & 15) == 0, "linear_umma: scale present iff int8");
  B200_REQUIRE(w24 == (w->meta != nullptr), "linear_umma: selectors present iff 2:4");
  B200_REQUIRE((w->k == D_MODEL && (w->ksplit == 4 || w->ksplit == 8)) || (w->k == 4 * D_MODEL && w->ksplit == 8),
               "linear_umma: K %d split %d ways", w->k, w->ksplit);
  B200_REQUIRE(w->n % UM == 0, "linear_umma: N %d", w->n);
  const b200dec_ln_link none{};
  const b200dec_ln_link lk = link ? *link : none;
  if (ln)
    B200_REQUIRE(a_kind == B200DEC_A_F16_ROWS16 && w->k == D_MODEL && w->ln_g && w->ln_bias && lk.stats_in &&
                     lk.stats_slots >= 1 && lk.stats_slots <= 128,
                 "linear_umma: LayerNorm rows come as a ready fp16 operand with partial sums");
  else
    B200_REQUIRE(a_kind == B200DEC_A_F16 || a_kind == B200DEC_A_F16_ROWS16, "linear_umma: fp16 rows only");
  B200_REQUIRE(rows >= 1 && rows <= 128 && lda % 8 == 0 && lda >= w->k && ldo % 4 == 0 && ((uintptr_t)a & 15) == 0 &&
                   ((uintptr_t)out & 15) == 0, "linear_umma: rows %d lda %d ldo %d", rows, lda, ldo);
  B200_REQUIRE(out_kind >= 0 && out_kind <= 2, "linear_umma: out_kind %d", out_kind);
  B200_REQUIRE(!lk.out16 || (out_kind == B200DEC_OUT_F32_ADD && lk.next_gamma && lk.stats_out),
               "linear_umma: the next LayerNorm's operand goes with OUT_F32_ADD, its gamma and the sums");
  // More than 64 rows: one 128-row tile per cluster (the wide K = 1024 projections), or the rows dealt over two
  // clusters of 64 rows per tile in the same launch (grid.z; the second reads the tile's weights from L2): K = 4096,
  // whose operands of 128 rows do not fit shared memory, and the 1024-wide projections, whose eight tiles would
  // otherwise make 64 CTAs.
  UArgs p{};
  p.w = (const uint8_t*)w->w, p.meta = (const uint32_t*)w->meta, p.scale = w->scale, p.bias = w->bias, p.xg = (const __half*)a;
  if (ln) {
    p.stats = lk.stats_in, p.stats_slots = lk.stats_slots;
    p.ln_g = w->ln_g, p.ln_bias = w->ln_bias, p.ln_eps = ln->eps;
  }
  p.out = out, p.status = status;
  if (lk.out16) p.next_gamma = lk.next_gamma, p.out16 = (__half*)lk.out16, p.stats_out = lk.stats_out;
  p.lda = lda, p.ldo = ldo, p.rows = rows, p.N = w->n, p.K = w->k;
  p.out_kind = out_kind, p.act = act;
  p.wait_limit = lk.wait_limit > 0 ? (uint32_t)lk.wait_limit : WAIT_LIMIT, p.withhold = lk.withhold;
  p.deal = rows > 64 && (w->k != D_MODEL || w->n <= D_MODEL);
  cudaStream_t s = (cudaStream_t)stream;
  const int wk = w16 ? 1 : w24 ? 2 : 0;
  if (w->k == D_MODEL && w->ksplit == 4) return launch_rows<4, 4>(p, wk, ln != nullptr, pdl, s);
  if (w->k == D_MODEL) return launch_rows<8, 2>(p, wk, ln != nullptr, pdl, s);
  return launch_rows<8, 8>(p, wk, false, pdl, s);
}

}  // namespace b200dec_detail

extern "C" int b200dec_tile_24_umma(const int8_t* kept, const int32_t* words, int n, int k, void* tiled, void* meta,
                                    void* stream) {
  B200_REQUIRE(kept && words && tiled && meta && n > 0 && n % UM == 0 && k > 0 && k % KB == 0,
               "tile_24_umma: (%d, %d) must be multiples of (128, 64)", n, k);
  const size_t total = (size_t)n * (k / 2);
  tile_24_umma_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      kept, (const uint32_t*)words, n, k, (uint8_t*)tiled, (uint32_t*)meta);
  return check_launch("tile_24_umma");
}
