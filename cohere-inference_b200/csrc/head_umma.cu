// Vocabulary projection with the final LayerNorm and a per-tile argmax on the fifth-generation tensor cores:
// logits(rows, N) = LayerNorm(x)(rows, 1024) . W(N, 1024)^T * scale + bias for rows <= 128, int8 weights.
//
// One CTA per 128 output channels and 64 rows (grid.y = 2 above 64 rows: the second set of CTAs finds its tiles'
// weights in L2), no split of K, no cluster: D(128 channels x 64 rows, fp32) lives in tensor memory
// and is accumulated by 64 `tcgen05.mma` instructions (M = 128, N = 64, K = 16, fp16 operands from shared memory).
//   * B operand: the CTA normalises all rows itself (it sees whole rows, so this is the plain two-pass LayerNorm, in
//     fp32) and writes them as fp16 into sixteen K-major tiles of 64 rows x 64 k with the 128-byte swizzle.
//   * A operand: the weights stream from HBM as 8 KB blocks (128 channels x 64 k, uint8 = q + 128, laid out by
//     b200dec_tile_int8_umma so that a thread's 16-byte pieces are conflict-free) through a ring filled by one
//     producer lane with cp.async.bulk; eight converter warps widen each block to fp16 (exact) into a second ring of
//     swizzled K-major tiles; one lane issues the MMAs of a block and `tcgen05.commit`s the tile's release.
//   * Epilogue: `tcgen05.ld` (thread = channel, 32 of the rows in registers), scale and bias, transposed through shared memory
//     for the per-row argmax over the CTA's channels (first index of the maximum, NaN never wins) and the optional
//     logits store.
// Every mbarrier wait is bounded; a wait that runs out sets B200DEC_ST_TIMEOUT and the roles fall through to the end
// (tensor memory is released on every path).
#include "common.cuh"

using namespace b200dec_detail;

namespace {

constexpr int UM = 128;                 // channels per CTA (MMA M)
constexpr int UN = 64;                  // rows (MMA N)
constexpr int KB = 64;                  // k per block: one 128-byte row of fp16
constexpr int NKB = D_MODEL / KB;       // 16 blocks
constexpr int RAW_STAGES = 7, A_STAGES = 2;  // 56 KB of weights in flight per SM (what fits beside the activations)
constexpr int RAW_BYTES = UM * KB;      // 8 KB of uint8
constexpr int A_BYTES = UM * KB * 2;    // 16 KB of fp16
constexpr int XB_BYTES = UN * KB * 2;   // 8 KB: one k-block of the activations
constexpr int X_BYTES = NKB * XB_BYTES; // 128 KB
constexpr int OFF_A = X_BYTES, OFF_RAW = OFF_A + A_STAGES * A_BYTES, SMEM_USED = OFF_RAW + RAW_STAGES * RAW_BYTES;
constexpr int SMEM_BYTES = SMEM_USED + 1024;  // slack to align the base to a swizzle atom
constexpr int OUT_LD = UM + 4;                // epilogue tile (64 rows x 128 channels fp32) row pitch, reuses the rings
static_assert(UN * OUT_LD * 4 <= SMEM_USED - OFF_A, "epilogue tile fits in the rings");
constexpr int NWORK = 8;                      // staging / converter / epilogue warps
constexpr int NTHREADS = (NWORK + 2) * 32;    // + the MMA warp and the producer warp
constexpr int TMEM_COLS = 64;
constexpr uint32_t WAIT_LIMIT = 1u << 22;

struct HeadArgs {
  const uint8_t* w;      // tiled weights
  const float* scale;
  const float* bias;     // may be null
  const float* x;        // (rows, lda) fp32, normalised in the kernel; or null:
  const __half* xg;      // (rows, lda) fp16 = row * gamma written by the projection that produced the rows, with
  const float* stats;    // (rows, stats_slots, 2) partial (sum, sum of squares); the LayerNorm is then folded into
  const float* ln_g;     // the epilogue: y = rstd * (acc * scale - mean * ln_g) + ln_bias + bias
  const float* ln_bias;
  int stats_slots;
  const float* ln_w;
  const float* ln_b;
  float* part_max;
  int* part_idx;
  float* logits;         // may be null
  int* status;
  float ln_eps;
  int lda, rows, N;
  uint32_t wait_limit;  // polls before a wait gives up
  int withhold;         // tests only: the producer stops after three blocks, so the waits behind it run out
};


DEVI uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
DEVI void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
DEVI void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
DEVI void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
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
DEVI void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
DEVI void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
DEVI void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
DEVI void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile with the 128-byte swizzle: rows of 128 bytes, groups of 8 rows
// 1024 bytes apart (the stride field), start address in 16-byte units, descriptor version 1, layout type 2.
DEVI uint64_t umma_desc(uint32_t saddr) {
  uint64_t d = (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;                  // leading-dimension offset: unused for a swizzled K-major tile
  d |= (uint64_t)(1024 >> 4) << 32;        // stride between 8-row groups
  d |= (uint64_t)1 << 46;                  // descriptor version
  d |= (uint64_t)2 << 61;                  // 128-byte swizzle
  return d;
}
// Instruction descriptor: fp16 x fp16 -> fp32, both operands K-major, N = 64, M = 128.
constexpr uint32_t UMMA_IDESC = (1u << 4) | ((uint32_t)(UN >> 3) << 17) | ((uint32_t)(UM >> 4) << 24);

DEVI void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(UMMA_IDESC), "r"(accumulate)
      : "memory");
}
template <uint32_t IDESC>
DEVI void umma_f16_n(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(da), "l"(db), "n"(IDESC), "r"(accumulate)
      : "memory");
}
DEVI void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// 16 values of uint8 = q + 128 -> 16 exact fp16 q (1024 + v as bits 0x6400 | v, minus 1152)
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

__global__ void __launch_bounds__(NTHREADS, 1) head_umma_kernel(const HeadArgs p_in) {
  // blockIdx.y: which 64 rows of the batch (rows 65-128 run as a second set of CTAs of the same launch: the tiles'
  // weights come from HBM once and from L2 for the other half)
  HeadArgs p = p_in;
  if (blockIdx.y > 0) {
    const int r0 = blockIdx.y * UN, np = p.N / UM;
    if (p.x) p.x += (size_t)r0 * p.lda;
    if (p.xg) p.xg += (size_t)r0 * p.lda, p.stats += (size_t)r0 * p.stats_slots * 2;
    p.part_max += (size_t)r0 * np, p.part_idx += (size_t)r0 * np;
    if (p.logits) p.logits += (size_t)r0 * p.N;
  }
  p.rows = p.rows - (int)blockIdx.y * UN < UN ? p.rows - (int)blockIdx.y * UN : UN;
  extern __shared__ unsigned char dyn_smem[];
  unsigned char* smem = dyn_smem + ((1024 - (smem_u32(dyn_smem) & 1023)) & 1023);  // swizzle atoms are 1 KB aligned
  unsigned char* xs = smem;
  unsigned char* as = smem + OFF_A;
  unsigned char* raws = smem + OFF_RAW;
  __shared__ __align__(8) uint64_t raw_full[RAW_STAGES], raw_empty[RAW_STAGES], a_full[A_STAGES], a_empty[A_STAGES];
  __shared__ __align__(8) uint64_t x_full, d_full;
  __shared__ uint32_t tmem_base;
  __shared__ float s_scale[UM], s_bias[UM], s_g[UM];
  __shared__ float s_mean[UN], s_rstd[UN];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x;  // channels [128 tile, +128)
  const uint8_t* wsrc = p.w + (size_t)tile * NKB * RAW_BYTES;

  if (tid == 0) {
    for (int i = 0; i < RAW_STAGES; ++i) mbar_init(&raw_full[i], 1), mbar_init(&raw_empty[i], NWORK);
    for (int i = 0; i < A_STAGES; ++i) mbar_init(&a_full[i], NWORK), mbar_init(&a_empty[i], 1);
    mbar_init(&x_full, NWORK), mbar_init(&d_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == NWORK) {  // the MMA warp owns the tensor memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base)),
                 "n"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid < UM) {
    s_scale[tid] = p.scale[tile * UM + tid];
    s_bias[tid] = (p.bias ? p.bias[tile * UM + tid] : 0.f) + (p.xg ? p.ln_bias[tile * UM + tid] : 0.f);
    s_g[tid] = p.xg ? p.ln_g[tile * UM + tid] : 0.f;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = tmem_base;

  if (warp == NWORK + 1) {
    // ---- producer: the tile's sixteen weight blocks through the raw ring (independent of the previous kernel) -------
    if (lane == 0) {
      bool ok = true;
      int issued = 0;
      for (int kb = 0; kb < NKB && ok; ++kb) {
        if (p.withhold && kb == 3) break;  // tests only: nothing sets the barriers of block 3
        const int st = kb % RAW_STAGES;
        ok = mbar_wait(&raw_empty[st], ((kb / RAW_STAGES) & 1) ^ 1, p.wait_limit);
        if (!ok) break;
        mbar_expect_tx(&raw_full[st], RAW_BYTES);
        bulk_load(raws + st * RAW_BYTES, wsrc + (size_t)kb * RAW_BYTES, RAW_BYTES, &raw_full[st]);
        issued = kb + 1;
      }
      if (!ok) {
        atomicOr(p.status, B200DEC_ST_TIMEOUT);
        // the copies already issued must land before this CTA's shared memory is given away (bounded)
        for (int kb = issued > RAW_STAGES ? issued - RAW_STAGES : 0; kb < issued; ++kb)
          mbar_wait(&raw_full[kb % RAW_STAGES], (kb / RAW_STAGES) & 1, p.wait_limit);
      }
    }
  } else if (warp == NWORK) {
    // ---- MMA issue: one lane, four instructions per block, the block's A tile released by the commit ---------------
    if (lane == 0) {
      bool ok = mbar_wait(&x_full, 0, p.wait_limit);
      for (int kb = 0; kb < NKB && ok; ++kb) {
        const int st = kb % A_STAGES;
        ok = mbar_wait(&a_full[st], (kb / A_STAGES) & 1, p.wait_limit);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a0 = smem_u32(as + st * A_BYTES), b0 = smem_u32(xs + kb * XB_BYTES);
#pragma unroll
        for (int k = 0; k < KB / 16; ++k)
          umma_f16(tmem_d, umma_desc(a0 + k * 32), umma_desc(b0 + k * 32), (kb | k) != 0);
        umma_commit(&a_empty[st]);
      }
      if (!ok) atomicOr(p.status, B200DEC_ST_TIMEOUT);
      umma_commit(&d_full);  // arrives when everything issued so far has completed (also after a time-out)
    }
  } else {
    // ---- workers: normalise the rows into the B tiles, then widen weight blocks, then the epilogue ------------------
    pdl_wait();
    pdl_trigger();
    if (p.xg) {
      // The operand exists already (row * gamma as fp16): 16-byte asynchronous copies straight into the swizzled
      // tiles, and the rows' statistics from the partial sums (four threads per row, fixed order).
      const int wt = tid;  // 0 .. 255
      for (int i = wt; i < UN * (D_MODEL / 8); i += NWORK * 32) {
        const int r = i >> 7, c = i & 127, kb = c >> 3, chunk = c & 7;  // row, 16-byte chunk of the row
        unsigned char* dst = xs + kb * XB_BYTES + (r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4);
        if (r < p.rows) cp_async16(dst, p.xg + (size_t)r * p.lda + c * 8);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
      }
      {
        const int r = wt >> 2, part = wt & 3;
        float s1 = 0.f, s2 = 0.f;
        if (r < p.rows) {
          const float2* ps = reinterpret_cast<const float2*>(p.stats) + (size_t)r * p.stats_slots;
          for (int i = part; i < p.stats_slots; i += 4) {
            const float2 v = __ldcg(ps + i);
            s1 += v.x, s2 += v.y;
          }
        }
        s1 += __shfl_xor_sync(0xffffffffu, s1, 1), s2 += __shfl_xor_sync(0xffffffffu, s2, 1);
        s1 += __shfl_xor_sync(0xffffffffu, s1, 2), s2 += __shfl_xor_sync(0xffffffffu, s2, 2);
        if (part == 0) {
          const float mean = s1 * (1.f / D_MODEL);
          s_mean[r] = mean;
          s_rstd[r] = rsqrtf(fmaxf(s2 * (1.f / D_MODEL) - mean * mean, 0.f) + p.ln_eps);
        }
      }
      cp_async_wait_all();
      asm volatile("bar.sync 1, %0;" ::"n"(NWORK * 32) : "memory");  // the statistics are read by other warps later
    } else
    // two rows per warp in flight (the loads of a row are one L2 round trip; a warp has 64 / 8 rows to do)
    for (int r0 = warp; r0 < UN; r0 += 2 * NWORK) {
      float v[2][32];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int r = (r0 + u * NWORK + tile) & (UN - 1);  // rotated by the tile index: at any moment the CTAs
        const bool live = r < p.rows;                       // of the grid ask L2 for different rows
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 f = live ? ld_cg_f4(p.x + (size_t)r * p.lda + i * 128 + lane * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
          v[u][4 * i] = f.x, v[u][4 * i + 1] = f.y, v[u][4 * i + 2] = f.z, v[u][4 * i + 3] = f.w;
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int r = (r0 + u * NWORK + tile) & (UN - 1);
        const bool live = r < p.rows;
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) s += v[u][i];
        const float mean = warp_sum(s) * (1.f / D_MODEL);
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) q += (v[u][i] - mean) * (v[u][i] - mean);
        const float rstd = rsqrtf(warp_sum(q) * (1.f / D_MODEL) + p.ln_eps);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int c = i * 128 + lane * 4;  // columns c .. c+3: half a 16-byte chunk of k-block c / 64
          const float4 g = __ldg(reinterpret_cast<const float4*>(p.ln_w + c));
          const float4 b = __ldg(reinterpret_cast<const float4*>(p.ln_b + c));
          uint2 h = make_uint2(0, 0);
          if (live)
            h = make_uint2(pack_f16((v[u][4 * i] - mean) * rstd * g.x + b.x, (v[u][4 * i + 1] - mean) * rstd * g.y + b.y),
                           pack_f16((v[u][4 * i + 2] - mean) * rstd * g.z + b.z,
                                    (v[u][4 * i + 3] - mean) * rstd * g.w + b.w));
          const int kb = c >> 6, chunk = (c & 63) >> 3;
          *reinterpret_cast<uint2*>(xs + kb * XB_BYTES + (r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4) +
                                    (c & 7) * 2) = h;
        }
      }
    }
    fence_async_shared();  // the MMA reads these tiles through the async proxy
    __syncwarp();
    if (lane == 0) mbar_arrive(&x_full);

    bool ok = true;
    const int ch = (warp & 3) * 32 + lane;  // this thread's channel of the tile (= its tensor-memory lane)
    const int hf = warp >> 2;               // and its half: 16-k pieces 2 hf, 2 hf + 1 of a block, rows 32 hf .. + 31
    for (int kb = 0; kb < NKB; ++kb) {
      if (!ok) break;
      const int rs = kb % RAW_STAGES, st = kb % A_STAGES;
      ok = mbar_wait(&raw_full[rs], (kb / RAW_STAGES) & 1, p.wait_limit);
      if (!ok) break;
      uint4 r[2];
#pragma unroll
      for (int j = 0; j < 2; ++j)
        r[j] = *reinterpret_cast<const uint4*>(raws + rs * RAW_BYTES + (2 * hf + j) * 2048 + ch * 16);
      __syncwarp();
      if (lane == 0) mbar_arrive(&raw_empty[rs]);  // the block's bytes are in registers
      ok = mbar_wait(&a_empty[st], ((kb / A_STAGES) & 1) ^ 1, p.wait_limit);
      if (!ok) break;
      unsigned char* row = as + st * A_BYTES + (ch >> 3) * 1024 + (ch & 7) * 128;
#pragma unroll
      for (int j = 0; j < 2; ++j) {  // piece pj: k = 16 pj .. 16 pj + 15 = chunks 2 pj and 2 pj + 1 of the row
        const int pj = 2 * hf + j;
        uint4 lo, hi;
        widen16(r[j], lo, hi);
        *reinterpret_cast<uint4*>(row + (((2 * pj) ^ (ch & 7)) << 4)) = lo;
        *reinterpret_cast<uint4*>(row + (((2 * pj + 1) ^ (ch & 7)) << 4)) = hi;
      }
      fence_async_shared();
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_full[st]);
    }
    if (!ok && lane == 0) atomicOr(p.status, B200DEC_ST_TIMEOUT);

    // ---- epilogue ---------------------------------------------------------------------------------------------------
    const bool got = mbar_wait(&d_full, 0, p.wait_limit);
    if (!got && lane == 0) atomicOr(p.status, B200DEC_ST_TIMEOUT);
    tc_fence_after();
    float* outs = reinterpret_cast<float*>(as);  // (64 rows, OUT_LD): the rings are idle once d_full has fired
    {
      uint32_t d[32];
      const uint32_t taddr = tmem_d + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(hf * 32);
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
      const float sc = s_scale[ch], bi = s_bias[ch], gch = s_g[ch];
      if (p.xg) {
#pragma unroll
        for (int r = 0; r < 32; ++r)
          outs[(hf * 32 + r) * OUT_LD + ch] =
              s_rstd[hf * 32 + r] * (__uint_as_float(d[r]) * sc - s_mean[hf * 32 + r] * gch) + bi;
      } else {
#pragma unroll
        for (int r = 0; r < 32; ++r) outs[(hf * 32 + r) * OUT_LD + ch] = __uint_as_float(d[r]) * sc + bi;
      }
    }
    tc_fence_before();
    asm volatile("bar.sync 1, %0;" ::"n"(NWORK * 32) : "memory");  // the workers only
    {
      // per-row argmax over the tile's channels: four threads per row, 32 channels each, lowest index wins ties
      const int r = tid >> 2, qt = tid & 3;
      float best = -INFINITY;
      int arg = 0x7fffffff;
      const float* rowp = outs + r * OUT_LD + qt * 32;
#pragma unroll 8
      for (int c = 0; c < 32; ++c) {
        const float v = rowp[c];
        if (v > best) best = v, arg = tile * UM + qt * 32 + c;
      }
#pragma unroll
      for (int o = 1; o < 4; o <<= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ob > best || (ob == best && oa < arg)) best = ob, arg = oa;
      }
      if (qt == 0 && r < p.rows) {
        const int np = p.N / UM;
        p.part_max[(size_t)r * np + tile] = best;
        p.part_idx[(size_t)r * np + tile] = arg;
      }
      if (p.logits) {
        for (int rr = warp; rr < p.rows; rr += NWORK)
          *reinterpret_cast<float4*>(p.logits + (size_t)rr * p.N + tile * UM + lane * 4) =
              *reinterpret_cast<const float4*>(outs + rr * OUT_LD + lane * 4);
      }
    }
  }
  // ---- release the tensor memory: after every warp is done with it ----------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == NWORK) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "n"(TMEM_COLS) : "memory");
  }
}

// ---- the same projection for the ready fp16 operand, streamed ------------------------------------------------------
//
// When the rows arrive as the finished operand (row * gamma in fp16, with their partial sums), nothing has to be
// normalised, so nothing has to be resident: the operand goes through a ring of k-blocks like the weights do. The
// 128 KB this frees go into (a) four weight-tile stages instead of two, so the workers hand over two blocks per turn
// (one proxy fence and one round of barrier traffic per pair; the clock stamps of the resident-operand kernel showed
// 880 cycles per block in the workers, a serial chain of waits, 100 instructions and a fence, against 130 for the
// block's four MMAs), and (b) 128 rows per CTA (MMA N = 128, 16 KB operand blocks), so a 65-128 row batch reads the
// weights once and runs as one wave of 128 CTAs instead of two sets of them.
// Operand block kb + LOOK is requested (cp.async, one commit group per block and thread) when block kb's weight tile
// is handed over; a thread waits for its own pieces of block kb just before that hand-over, so the MMA lane's wait on
// the tile's barrier covers the operand block as well, and the commit that frees weight stage kb also frees operand
// stage kb (XS = LOOK + AST stages: block kb + LOOK reuses the stage of block kb - AST).
// The rows' statistics: a warp per row, the row's partial sums read with coalesced loads that are all in flight at
// once (four threads per row walking 128 slots one after the other took 3.5 us of the resident-operand kernel).
// fp16 weights (W16, kind B200DEC_W_F16_UMMA) are stored as the images of the swizzled weight tiles: the producer lane
// copies a block from HBM straight into a weight stage (`cp.async.bulk`, the stage's barrier counts its bytes beside
// the workers' arrivals for the operand block), there is no raw ring and no widening, the shared memory that ring took
// holds more weight stages (9 or 7 blocks of 16 KB in flight), and the operand stages are freed by a commit of their
// own.
template <int UNS, bool W16>
struct HeadStream {
  static constexpr int AST = W16 ? (UNS == 64 ? 9 : 7) : 4;  // weight-tile stages
  static constexpr int NWK = 16;                     // worker warps: one 16-byte piece of a weight block per thread
  static constexpr int NT = (NWK + 2) * 32;          // + the MMA warp and the producer warp
  static constexpr int LOOK = UNS == 64 ? 4 : 2;     // operand blocks requested ahead
  static constexpr int XS = LOOK + 4;                // int8: block kb + LOOK reuses the stage of block kb - AST
  static constexpr int XB = UNS * KB * 2;            // one k-block of the operand: 8 or 16 KB
  static constexpr int RAW = W16 ? 0 : UNS == 64 ? 10 : 7;  // raw weight blocks in flight: what fits beside the other rings
  static constexpr int OFF_X = 0, OFF_A = XS * XB, OFF_RAW = OFF_A + AST * A_BYTES, USED = OFF_RAW + RAW * RAW_BYTES;
  static constexpr int BYTES = USED + 1024;
  static constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(UNS >> 3) << 17) | ((uint32_t)(UM >> 4) << 24);
  static_assert(UNS * OUT_LD * 4 <= USED - OFF_A, "epilogue tile fits in the weight rings");
  static_assert(BYTES + 4096 <= 227 * 1024, "rings + static shared memory fit an SM");
  static_assert(W16 || (NKB % 2 == 0 && AST % 2 == 0 && XS == LOOK + AST), "the workers hand over blocks in pairs");
  static_assert(!W16 || AST > XS - LOOK, "a weight stage's previous use is over before the workers arrive for the next");
};

template <int UNS, bool W16>
__global__ void __launch_bounds__(HeadStream<UNS, W16>::NT, 1) head_stream_kernel(const HeadArgs p) {
  using C = HeadStream<UNS, W16>;
  constexpr int RS = W16 ? 1 : C::RAW, LOOK = C::LOOK, XS = C::XS, AST = C::AST, NWK = C::NWK;
  extern __shared__ unsigned char dyn_smem[];
  unsigned char* smem = dyn_smem + ((1024 - (smem_u32(dyn_smem) & 1023)) & 1023);  // swizzle atoms are 1 KB aligned
  unsigned char* xs = smem + C::OFF_X;
  unsigned char* as = smem + C::OFF_A;
  unsigned char* raws = smem + C::OFF_RAW;
  __shared__ __align__(8) uint64_t raw_full[RS], raw_empty[RS], a_full[AST], a_empty[AST], x_empty[XS];
  __shared__ __align__(8) uint64_t d_full;
  __shared__ uint32_t tmem_base;
  __shared__ float s_scale[UM], s_bias[UM], s_g[UM];
  __shared__ float s_mean[UNS], s_rstd[UNS];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x;  // channels [128 tile, +128)
  const uint8_t* wsrc = p.w + (size_t)tile * NKB * (W16 ? A_BYTES : RAW_BYTES);

  if (tid == 0) {
    for (int i = 0; i < RS; ++i) mbar_init(&raw_full[i], 1), mbar_init(&raw_empty[i], NWK);
    // fp16 weights: a stage is full when the workers' operand pieces and the producer's bytes are there
    for (int i = 0; i < AST; ++i) mbar_init(&a_full[i], W16 ? NWK + 1 : NWK), mbar_init(&a_empty[i], 1);
    for (int i = 0; i < XS; ++i) mbar_init(&x_empty[i], 1);
    mbar_init(&d_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == NWK) {  // the MMA warp owns the tensor memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base)),
                 "n"(UNS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid < UM) {
    s_scale[tid] = p.scale ? p.scale[tile * UM + tid] : 1.f;
    s_bias[tid] = (p.bias ? p.bias[tile * UM + tid] : 0.f) + p.ln_bias[tile * UM + tid];
    s_g[tid] = p.ln_g[tile * UM + tid];
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = tmem_base;

  if (warp == NWK + 1) {
    // ---- producer: the tile's sixteen weight blocks through the raw ring, or (fp16) straight into the weight stages
    // (independent of the previous kernel) ------------------------------------------------------------------------------
    if (lane == 0) {
      constexpr int PS = W16 ? AST : RS;                      // the ring the producer fills
      constexpr uint32_t PB = W16 ? A_BYTES : RAW_BYTES;      // bytes per block
      uint64_t* full = W16 ? a_full : raw_full;
      uint64_t* empty = W16 ? a_empty : raw_empty;
      unsigned char* ring = W16 ? as : raws;
      bool ok = true;
      int issued = 0;
      for (int kb = 0; kb < NKB && ok; ++kb) {
        if (p.withhold && kb == 3) break;  // tests only: nothing sets the barriers of block 3
        const int st = kb % PS;
        ok = mbar_wait(&empty[st], ((kb / PS) & 1) ^ 1, p.wait_limit);
        if (!ok) break;
        mbar_expect_tx(&full[st], PB);
        bulk_load(ring + st * PB, wsrc + (size_t)kb * PB, PB, &full[st]);
        issued = kb + 1;
      }
      if (!ok) {
        atomicOr(p.status, B200DEC_ST_TIMEOUT);
        for (int kb = issued > PS ? issued - PS : 0; kb < issued; ++kb)  // copies in flight land before the CTA leaves
          mbar_wait(&full[kb % PS], (kb / PS) & 1, p.wait_limit);
      }
    }
  } else if (warp == NWK) {
    // ---- MMA issue: one lane; a block's barrier stands for its weight tile and its operand block ------------------
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < NKB && ok; ++kb) {
        const int st = kb % AST;
        ok = mbar_wait(&a_full[st], (kb / AST) & 1, p.wait_limit);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a0 = smem_u32(as + st * A_BYTES), b0 = smem_u32(xs + (kb % XS) * C::XB);
#pragma unroll
        for (int k = 0; k < KB / 16; ++k)
          umma_f16_n<C::IDESC>(tmem_d, umma_desc(a0 + k * 32), umma_desc(b0 + k * 32), (kb | k) != 0);
        umma_commit(&a_empty[st]);
        if constexpr (W16) umma_commit(&x_empty[kb % XS]);
      }
      if (!ok) atomicOr(p.status, B200DEC_ST_TIMEOUT);
      umma_commit(&d_full);  // arrives when everything issued so far has completed (also after a time-out)
    }
  } else {
    // ---- workers: request operand blocks, widen weight blocks, then the epilogue ------------------------------------
    pdl_wait();
    pdl_trigger();
    auto request_x = [&](int kb) {  // this thread's 16-byte pieces of operand block kb; always one commit group
      if (kb < NKB) {
        unsigned char* xb = xs + (kb % XS) * C::XB;
        for (int i = tid; i < UNS * 8; i += NWK * 32) {
          const int r = i >> 3, chunk = i & 7;
          unsigned char* dst = xb + (r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4);
          if (r < p.rows) cp_async16(dst, p.xg + (size_t)r * p.lda + kb * KB + chunk * 8);
          else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
      }
      cp_async_commit();
    };
#pragma unroll
    for (int kb = 0; kb < LOOK; ++kb) request_x(kb);
    // the rows' statistics from the partial sums (at most 128 per row): a warp per row, all of a warp's loads at once
    {
      constexpr int RPW = UNS / NWK;  // 4 or 8 rows per warp
      float2 v[RPW][4];
#pragma unroll
      for (int j = 0; j < RPW; ++j) {
        const int r = warp + NWK * j;
        const float2* ps = reinterpret_cast<const float2*>(p.stats) + (size_t)r * p.stats_slots;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          v[j][i] = (r < p.rows && lane + 32 * i < p.stats_slots) ? __ldcg(ps + lane + 32 * i) : make_float2(0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < RPW; ++j) {
        const int r = warp + NWK * j;
        float s1 = (v[j][0].x + v[j][1].x) + (v[j][2].x + v[j][3].x), s2 = (v[j][0].y + v[j][1].y) + (v[j][2].y + v[j][3].y);
        s1 = warp_sum(s1), s2 = warp_sum(s2);
        if (lane == 0) {
          const float mean = s1 * (1.f / D_MODEL);
          s_mean[r] = mean;
          s_rstd[r] = rsqrtf(fmaxf(s2 * (1.f / D_MODEL) - mean * mean, 0.f) + p.ln_eps);
        }
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(NWK * 32) : "memory");  // the statistics are read by other warps later

    bool ok = true;
    const int ch = (warp & 3) * 32 + lane;  // this thread's channel of the tile (= its tensor-memory lane)
    const int pj = warp >> 2;               // and its quarter: the 16-k piece pj of a block, rows pj * UNS / 4 .. after
    if constexpr (W16) {
      // fp16 weights: the workers only keep the operand ring LOOK blocks ahead and vouch for their pieces of block kb
      for (int kb = 0; kb < NKB; ++kb) {
        const int nb = kb + LOOK;
        if (nb < NKB && nb >= XS)  // the MMAs of block nb - XS, the stage's previous tenant, are done
          ok = mbar_wait(&x_empty[nb % XS], ((nb / XS) - 1) & 1, p.wait_limit);
        if (!ok) break;
        request_x(nb);
        cp_async_wait_group<LOOK>();  // this thread's pieces of operand block kb (and earlier) have landed
        fence_async_shared();
        __syncwarp();
        if (lane == 0) mbar_arrive(&a_full[kb % AST]);
      }
    } else {
      for (int kb = 0; kb < NKB && ok; kb += 2) {  // two blocks per turn
        uint4 r[2];
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const int rs = (kb + b) % RS;
          ok = ok && mbar_wait(&raw_full[rs], ((kb + b) / RS) & 1, p.wait_limit);
          if (ok) r[b] = *reinterpret_cast<const uint4*>(raws + rs * RAW_BYTES + pj * 2048 + ch * 16);
        }
        if (!ok) break;
        __syncwarp();
        if (lane == 0) mbar_arrive(&raw_empty[kb % RS]), mbar_arrive(&raw_empty[(kb + 1) % RS]);  // bytes are in registers
        // MMAs of blocks kb - AST and kb + 1 - AST are done: their weight and operand stages are free
#pragma unroll
        for (int b = 0; b < 2; ++b)
          ok = ok && mbar_wait(&a_empty[(kb + b) % AST], (((kb + b) / AST) & 1) ^ 1, p.wait_limit);
        if (!ok) break;
        request_x(kb + LOOK);
        request_x(kb + 1 + LOOK);
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          unsigned char* row = as + ((kb + b) % AST) * A_BYTES + (ch >> 3) * 1024 + (ch & 7) * 128;
          uint4 lo, hi;  // piece pj: k = 16 pj .. 16 pj + 15 = chunks 2 pj and 2 pj + 1 of the row
          widen16(r[b], lo, hi);
          *reinterpret_cast<uint4*>(row + (((2 * pj) ^ (ch & 7)) << 4)) = lo;
          *reinterpret_cast<uint4*>(row + (((2 * pj + 1) ^ (ch & 7)) << 4)) = hi;
        }
        cp_async_wait_group<LOOK>();  // this thread's pieces of operand blocks kb and kb + 1 (and earlier) have landed
        fence_async_shared();
        __syncwarp();
        if (lane == 0) mbar_arrive(&a_full[kb % AST]), mbar_arrive(&a_full[(kb + 1) % AST]);
      }
    }
    cp_async_wait_all();  // nothing of this thread's is on its way into the rings any more (also after a time-out)
    if (!ok && lane == 0) atomicOr(p.status, B200DEC_ST_TIMEOUT);

    // ---- epilogue ---------------------------------------------------------------------------------------------------
    const bool got = mbar_wait(&d_full, 0, p.wait_limit);
    if (!got && lane == 0) atomicOr(p.status, B200DEC_ST_TIMEOUT);
    tc_fence_after();
    float* outs = reinterpret_cast<float*>(as);  // (UNS rows, OUT_LD): the weight rings are idle once d_full has fired
    const float sc = s_scale[ch], bi = s_bias[ch], gch = s_g[ch];
    {
      constexpr int CW = UNS / 4;  // accumulator columns (= rows) per warp: 16 or 32
      uint32_t d[CW];
      const int row0 = pj * CW;
      const uint32_t taddr = tmem_d + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)row0;
      if constexpr (CW == 32) {
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
      } else {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]), "=r"(d[8]),
              "=r"(d[9]), "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15])
            : "r"(taddr)
            : "memory");
      }
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
      for (int r = 0; r < CW; ++r)
        outs[(row0 + r) * OUT_LD + ch] = s_rstd[row0 + r] * (__uint_as_float(d[r]) * sc - s_mean[row0 + r] * gch) + bi;
    }
    tc_fence_before();
    asm volatile("bar.sync 1, %0;" ::"n"(NWK * 32) : "memory");  // the workers only
    // per-row argmax over the tile's channels: four threads per row, 32 channels each, lowest index wins ties
    if (tid < UNS * 4) {
      const int r = tid >> 2, qt = tid & 3;  // the shuffles below stay inside a row's four lanes
      float best = -INFINITY;
      int arg = 0x7fffffff;
      const float* rowp = outs + r * OUT_LD + qt * 32;
#pragma unroll 8
      for (int c = 0; c < 32; ++c) {
        const float v = rowp[c];
        if (v > best) best = v, arg = tile * UM + qt * 32 + c;
      }
#pragma unroll
      for (int o = 1; o < 4; o <<= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ob > best || (ob == best && oa < arg)) best = ob, arg = oa;
      }
      if (qt == 0 && r < p.rows) {
        const int np = p.N / UM;
        p.part_max[(size_t)r * np + tile] = best;
        p.part_idx[(size_t)r * np + tile] = arg;
      }
    }
    if (p.logits) {
      for (int rr = warp; rr < p.rows; rr += NWK)
        *reinterpret_cast<float4*>(p.logits + (size_t)rr * p.N + tile * UM + lane * 4) =
            *reinterpret_cast<const float4*>(outs + rr * OUT_LD + lane * 4);
    }
  }
  // ---- release the tensor memory: after every warp is done with it ----------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == NWK) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "n"(UNS) : "memory");
  }
}

// w (n, k) 16-bit row-major -> blocks [n / 128][k / 64] of 16 KB, each the image of a K-major tile with the 128-byte
// swizzle: channel t's 128-byte row at 128 t, its 16-byte chunk c (k = 8 c .. 8 c + 7 of the block) at position c ^ (t & 7)
__global__ void tile_f16_umma_kernel(const uint16_t* __restrict__ w, int n, int k, uint16_t* __restrict__ out) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // one output element each
  if (i >= (size_t)n * k) return;
  const int e = i & 7, pos = (i >> 3) & 7, t = (i >> 6) & 127;
  const size_t blk = i >> 13;
  const int nkb = k / KB, kb = (int)(blk % nkb), mt = (int)(blk / nkb), c = pos ^ (t & 7);
  out[i] = w[(size_t)(mt * UM + t) * k + kb * KB + c * 8 + e];
}

// q (n, k) int8 row-major -> blocks [n / 128][k / 64] of 8 KB: [16-k piece j = 0..3][channel t = 0..127][16 bytes],
// bytes = q + 128
__global__ void tile_int8_umma_kernel(const int8_t* __restrict__ q, int n, int k, uint8_t* __restrict__ out) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // one output byte each
  if (i >= (size_t)n * k) return;
  const int e = i & 15, t = (i >> 4) & 127, j = (i >> 11) & 3;
  const size_t blk = i >> 13;
  const int nkb = k / KB, kb = (int)(blk % nkb), mt = (int)(blk / nkb);
  out[i] = (uint8_t)((int)q[(size_t)(mt * UM + t) * k + kb * KB + j * 16 + e] + 128);
}

}  // namespace

namespace b200dec_detail {

// x: fp32 rows normalised by the kernel (xg null), or xg: the ready fp16 operand (row * gamma) with its partial sums
// (x null; w->ln_g / ln_bias fold the LayerNorm into the epilogue).
int head_umma_impl(const b200dec_weight* w, const float* x, const void* xg, const float* stats, int stats_slots,
                   const b200dec_norm* ln, int lda, int rows, float* part_max, int32_t* part_idx, float* logits,
                   int32_t* status, int pdl, void* stream, int wait_limit, int withhold) {
  B200_REQUIRE(w && w->w && (x || xg) && ln && ln->w && ln->b && part_max && part_idx && status,
               "head_umma: null pointer");
  const bool w16 = w->kind == B200DEC_W_F16_UMMA;
  B200_REQUIRE(w16 == (w->scale == nullptr) && ((uintptr_t)w->w & 15) == 0, "head_umma: scale present iff int8");
  B200_REQUIRE(!w16 || xg, "head_umma: fp16 weights take the ready fp16 operand (b200dec_head_umma_linked)");
  B200_REQUIRE(!xg || (stats && stats_slots >= 1 && w->ln_g && w->ln_bias && ((uintptr_t)xg & 15) == 0 && lda % 8 == 0),
               "head_umma: the fp16 operand comes with its partial sums and the weight's ln_g / ln_bias");
  B200_REQUIRE((w->kind == B200DEC_W_INT8_UMMA || w16) && w->k == D_MODEL && w->n % UM == 0, "head_umma: weight kind %d (%d, %d)",
               w->kind, w->n, w->k);
  B200_REQUIRE(rows >= 1 && rows <= 128 && lda % 4 == 0 && ((uintptr_t)x & 15) == 0, "head_umma: rows %d lda %d", rows,
               lda);
  if (xg) x = nullptr;
  cudaError_t e = cudaFuncSetAttribute(head_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "head_umma: smem attribute: %s", cudaGetErrorString(e));
  const int np = w->n / UM;
  HeadArgs a{};
  a.w = (const uint8_t*)w->w, a.scale = w->scale, a.bias = w->bias, a.x = x;
  if (xg) {
    a.xg = (const __half*)xg, a.stats = stats;
    a.stats_slots = stats_slots, a.ln_g = w->ln_g, a.ln_bias = w->ln_bias;
  }
  a.ln_w = ln->w, a.ln_b = ln->b, a.ln_eps = ln->eps;
  a.part_max = part_max, a.part_idx = part_idx, a.logits = logits;
  a.status = status, a.lda = lda, a.rows = rows, a.N = w->n;
  a.wait_limit = wait_limit > 0 ? (uint32_t)wait_limit : WAIT_LIMIT, a.withhold = withhold;
  if (xg) {  // the ready operand: streamed, one CTA per tile whatever the rows (at most 128 partial sums per row)
    B200_REQUIRE(stats_slots <= 128, "head_umma: %d partial sums per row (at most 128)", stats_slots);
    auto go = [&](auto kern, int threads, int bytes) {
      cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
      return err != cudaSuccess ? err : launch_kernel(kern, dim3(np), dim3(threads), bytes, (cudaStream_t)stream, 0, pdl, a);
    };
    if (rows <= UN)
      e = w16 ? go(head_stream_kernel<64, true>, HeadStream<64, true>::NT, HeadStream<64, true>::BYTES)
              : go(head_stream_kernel<64, false>, HeadStream<64, false>::NT, HeadStream<64, false>::BYTES);
    else
      e = w16 ? go(head_stream_kernel<128, true>, HeadStream<128, true>::NT, HeadStream<128, true>::BYTES)
              : go(head_stream_kernel<128, false>, HeadStream<128, false>::NT, HeadStream<128, false>::BYTES);
    if (e != cudaSuccess) return fail(B200DEC_ECUDA, "head_umma (streamed operand) launch: %s", cudaGetErrorString(e));
    return 0;
  }
  // fp32 rows that the CTA normalises: the operand resident, a set of CTAs per 64 rows (the kernel offsets its rows
  // by blockIdx.y)
  e = launch_kernel(head_umma_kernel, dim3(np, (rows + UN - 1) / UN), dim3(NTHREADS), SMEM_BYTES, (cudaStream_t)stream, 0,
                    pdl, a);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "head_umma launch: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace b200dec_detail

extern "C" {

int b200dec_tile_int8_umma(const int8_t* q, int n, int k, void* tiled, void* stream) {
  B200_REQUIRE(q && tiled && n > 0 && n % UM == 0 && k > 0 && k % KB == 0, "tile_int8_umma: (%d, %d) must be multiples of (128, 64)",
               n, k);
  const size_t total = (size_t)n * k;
  tile_int8_umma_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(q, n, k, (uint8_t*)tiled);
  return check_launch("tile_int8_umma");
}

int b200dec_tile_f16_umma(const void* w16, int n, int k, void* tiled, void* stream) {
  B200_REQUIRE(w16 && tiled && n > 0 && n % UM == 0 && k > 0 && k % KB == 0, "tile_f16_umma: (%d, %d) must be multiples of (128, 64)",
               n, k);
  const size_t total = (size_t)n * k;
  tile_f16_umma_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const uint16_t*)w16, n, k,
                                                                                          (uint16_t*)tiled);
  return check_launch("tile_f16_umma");
}

int b200dec_head_umma(const b200dec_weight* w, const float* x, const b200dec_norm* ln, int lda, int rows,
                      float* part_max, int32_t* part_idx, float* logits, int32_t* status, int pdl, void* stream) {
  return head_umma_impl(w, x, nullptr, nullptr, 0, ln, lda, rows, part_max, part_idx, logits, status, pdl, stream, 0, 0);
}

int b200dec_head_umma_linked(const b200dec_weight* w, const void* xg, const float* stats, int stats_slots,
                             const b200dec_norm* ln, int lda, int rows, float* part_max, int32_t* part_idx,
                             float* logits, int32_t* status, int pdl, void* stream) {
  B200_REQUIRE(xg, "head_umma_linked: null operand");
  return head_umma_impl(w, nullptr, xg, stats, stats_slots, ln, lda, rows, part_max, part_idx, logits, status, pdl,
                        stream, 0, 0);
}

}  // extern "C"
