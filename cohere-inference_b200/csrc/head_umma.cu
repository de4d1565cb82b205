// Vocabulary projection with the final LayerNorm and a per-tile argmax on the fifth-generation tensor cores:
// logits(rows, N) = LayerNorm(x)(rows, 1024) . W(N, 1024)^T * scale + bias for rows <= 64, int8 weights.
//
// One CTA per 128 output channels, no split of K, no cluster: D(128 channels x 64 rows, fp32) lives in tensor memory
// and is accumulated by 64 `tcgen05.mma` instructions (M = 128, N = 64, K = 16, fp16 operands from shared memory).
//   * B operand: the CTA normalises all rows itself (it sees whole rows, so this is the plain two-pass LayerNorm, in
//     fp32) and writes them as fp16 into sixteen K-major tiles of 64 rows x 64 k with the 128-byte swizzle.
//   * A operand: the weights stream from HBM as 8 KB blocks (128 channels x 64 k, uint8 = q + 128, laid out by
//     b200dec_tile_int8_umma so that a thread's 16-byte pieces are conflict-free) through a ring filled by one
//     producer lane with cp.async.bulk; four converter warps widen each block to fp16 (exact) into a second ring of
//     swizzled K-major tiles; one lane issues the MMAs of a block and `tcgen05.commit`s the tile's release.
//   * Epilogue: `tcgen05.ld` (thread = channel, 64 rows in registers), scale and bias, transposed through shared memory
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
constexpr int RAW_STAGES = 4, A_STAGES = 3;
constexpr int RAW_BYTES = UM * KB;      // 8 KB of uint8
constexpr int A_BYTES = UM * KB * 2;    // 16 KB of fp16
constexpr int XB_BYTES = UN * KB * 2;   // 8 KB: one k-block of the activations
constexpr int X_BYTES = NKB * XB_BYTES; // 128 KB
constexpr int OFF_A = X_BYTES, OFF_RAW = OFF_A + A_STAGES * A_BYTES, SMEM_USED = OFF_RAW + RAW_STAGES * RAW_BYTES;
constexpr int SMEM_BYTES = SMEM_USED + 1024;  // slack to align the base to a swizzle atom
constexpr int OUT_LD = UM + 4;                // epilogue tile (64 rows x 128 channels fp32) row pitch, reuses the rings
static_assert(UN * OUT_LD * 4 <= SMEM_USED - OFF_A, "epilogue tile fits in the rings");
constexpr int NWORK = 4;                      // converter / epilogue warps
constexpr int NTHREADS = (NWORK + 2) * 32;    // + the MMA warp and the producer warp
constexpr int TMEM_COLS = 64;
constexpr uint32_t WAIT_LIMIT = 1u << 22;

struct HeadArgs {
  const uint8_t* w;      // tiled weights
  const float* scale;
  const float* bias;     // may be null
  const float* x;        // (rows, lda) fp32
  const float* ln_w;
  const float* ln_b;
  float* part_max;
  int* part_idx;
  float* logits;         // may be null
  int* status;
  float ln_eps;
  int lda, rows, N;
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
DEVI bool mbar_wait(uint64_t* bar, uint32_t parity) {  // bounded; false when the limit ran out
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
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

__global__ void __launch_bounds__(NTHREADS, 1) head_umma_kernel(const HeadArgs p) {
  extern __shared__ unsigned char dyn_smem[];
  unsigned char* smem = dyn_smem + ((1024 - (smem_u32(dyn_smem) & 1023)) & 1023);  // swizzle atoms are 1 KB aligned
  unsigned char* xs = smem;
  unsigned char* as = smem + OFF_A;
  unsigned char* raws = smem + OFF_RAW;
  __shared__ __align__(8) uint64_t raw_full[RAW_STAGES], raw_empty[RAW_STAGES], a_full[A_STAGES], a_empty[A_STAGES];
  __shared__ __align__(8) uint64_t x_full, d_full;
  __shared__ uint32_t tmem_base;
  __shared__ float s_scale[UM], s_bias[UM];

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
    s_bias[tid] = p.bias ? p.bias[tile * UM + tid] : 0.f;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = tmem_base;

  if (warp == NWORK + 1) {
    // ---- producer: the tile's sixteen weight blocks through the raw ring (independent of the previous kernel) -------
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < NKB && ok; ++kb) {
        const int st = kb % RAW_STAGES;
        ok = mbar_wait(&raw_empty[st], ((kb / RAW_STAGES) & 1) ^ 1);
        if (!ok) break;
        mbar_expect_tx(&raw_full[st], RAW_BYTES);
        bulk_load(raws + st * RAW_BYTES, wsrc + (size_t)kb * RAW_BYTES, RAW_BYTES, &raw_full[st]);
      }
      if (!ok) atomicOr(p.status, B200DEC_ST_TIMEOUT);
    }
  } else if (warp == NWORK) {
    // ---- MMA issue: one lane, four instructions per block, the block's A tile released by the commit ---------------
    if (lane == 0) {
      bool ok = mbar_wait(&x_full, 0);
      for (int kb = 0; kb < NKB && ok; ++kb) {
        const int st = kb % A_STAGES;
        ok = mbar_wait(&a_full[st], (kb / A_STAGES) & 1);
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
    for (int r = warp; r < UN; r += NWORK) {
      float v[32];
      const bool live = r < p.rows;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 f = live ? ld_cg_f4(p.x + (size_t)r * p.lda + i * 128 + lane * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        v[4 * i] = f.x, v[4 * i + 1] = f.y, v[4 * i + 2] = f.z, v[4 * i + 3] = f.w;
      }
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) s += v[i];
      const float mean = warp_sum(s) * (1.f / D_MODEL);
      float q = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) q += (v[i] - mean) * (v[i] - mean);
      const float rstd = rsqrtf(warp_sum(q) * (1.f / D_MODEL) + p.ln_eps);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int c = i * 128 + lane * 4;  // columns c .. c+3: half a 16-byte chunk of k-block c / 64
        const float4 g = __ldg(reinterpret_cast<const float4*>(p.ln_w + c));
        const float4 b = __ldg(reinterpret_cast<const float4*>(p.ln_b + c));
        uint2 h = make_uint2(0, 0);
        if (live)
          h = make_uint2(pack_f16((v[4 * i] - mean) * rstd * g.x + b.x, (v[4 * i + 1] - mean) * rstd * g.y + b.y),
                         pack_f16((v[4 * i + 2] - mean) * rstd * g.z + b.z, (v[4 * i + 3] - mean) * rstd * g.w + b.w));
        const int kb = c >> 6, chunk = (c & 63) >> 3;
        *reinterpret_cast<uint2*>(xs + kb * XB_BYTES + (r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4) +
                                  (c & 7) * 2) = h;
      }
    }
    fence_async_shared();  // the MMA reads these tiles through the async proxy
    __syncwarp();
    if (lane == 0) mbar_arrive(&x_full);

    bool ok = true;
    const int ch = tid;  // this thread's channel of the tile
    for (int kb = 0; kb < NKB; ++kb) {
      if (!ok) break;
      const int rs = kb % RAW_STAGES, st = kb % A_STAGES;
      ok = mbar_wait(&raw_full[rs], (kb / RAW_STAGES) & 1);
      if (!ok) break;
      uint4 r[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) r[j] = *reinterpret_cast<const uint4*>(raws + rs * RAW_BYTES + j * 2048 + ch * 16);
      __syncwarp();
      if (lane == 0) mbar_arrive(&raw_empty[rs]);  // the block's bytes are in registers
      ok = mbar_wait(&a_empty[st], ((kb / A_STAGES) & 1) ^ 1);
      if (!ok) break;
      unsigned char* row = as + st * A_BYTES + (ch >> 3) * 1024 + (ch & 7) * 128;
#pragma unroll
      for (int j = 0; j < 4; ++j) {  // k = 16 j .. 16 j + 15: chunks 2j and 2j + 1 of the row
        uint4 lo, hi;
        widen16(r[j], lo, hi);
        *reinterpret_cast<uint4*>(row + (((2 * j) ^ (ch & 7)) << 4)) = lo;
        *reinterpret_cast<uint4*>(row + (((2 * j + 1) ^ (ch & 7)) << 4)) = hi;
      }
      fence_async_shared();
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_full[st]);
    }
    if (!ok && lane == 0) atomicOr(p.status, B200DEC_ST_TIMEOUT);

    // ---- epilogue ---------------------------------------------------------------------------------------------------
    const bool got = mbar_wait(&d_full, 0);
    if (!got && lane == 0) atomicOr(p.status, B200DEC_ST_TIMEOUT);
    tc_fence_after();
    float* outs = reinterpret_cast<float*>(as);  // (64 rows, OUT_LD): the rings are idle once d_full has fired
    {
      uint32_t d[UN];
      const uint32_t taddr = tmem_d + ((uint32_t)(warp * 32) << 16);
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
          "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
          "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
          "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
          "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
          : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(d[6]), "=r"(d[7]), "=r"(d[8]),
            "=r"(d[9]), "=r"(d[10]), "=r"(d[11]), "=r"(d[12]), "=r"(d[13]), "=r"(d[14]), "=r"(d[15]), "=r"(d[16]),
            "=r"(d[17]), "=r"(d[18]), "=r"(d[19]), "=r"(d[20]), "=r"(d[21]), "=r"(d[22]), "=r"(d[23]), "=r"(d[24]),
            "=r"(d[25]), "=r"(d[26]), "=r"(d[27]), "=r"(d[28]), "=r"(d[29]), "=r"(d[30]), "=r"(d[31]), "=r"(d[32]),
            "=r"(d[33]), "=r"(d[34]), "=r"(d[35]), "=r"(d[36]), "=r"(d[37]), "=r"(d[38]), "=r"(d[39]), "=r"(d[40]),
            "=r"(d[41]), "=r"(d[42]), "=r"(d[43]), "=r"(d[44]), "=r"(d[45]), "=r"(d[46]), "=r"(d[47]), "=r"(d[48]),
            "=r"(d[49]), "=r"(d[50]), "=r"(d[51]), "=r"(d[52]), "=r"(d[53]), "=r"(d[54]), "=r"(d[55]), "=r"(d[56]),
            "=r"(d[57]), "=r"(d[58]), "=r"(d[59]), "=r"(d[60]), "=r"(d[61]), "=r"(d[62]), "=r"(d[63])
          : "r"(taddr)
          : "memory");
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      const float sc = s_scale[ch], bi = s_bias[ch];
#pragma unroll
      for (int r = 0; r < UN; ++r) outs[r * OUT_LD + ch] = __uint_as_float(d[r]) * sc + bi;
    }
    tc_fence_before();
    asm volatile("bar.sync 1, %0;" ::"n"(NWORK * 32) : "memory");  // the workers only
    {
      // per-row argmax over the tile's channels: two threads per row, 64 channels each, lowest index wins ties
      const int r = tid >> 1, half = tid & 1;
      float best = -INFINITY;
      int arg = 0x7fffffff;
      const float* rowp = outs + r * OUT_LD + half * 64;
#pragma unroll 8
      for (int c = 0; c < 64; ++c) {
        const float v = rowp[c];
        if (v > best) best = v, arg = tile * UM + half * 64 + c;
      }
      const float ob = __shfl_xor_sync(0xffffffffu, best, 1);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, 1);
      if (ob > best || (ob == best && oa < arg)) best = ob, arg = oa;
      if (half == 0 && r < p.rows) {
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

int head_umma_impl(const b200dec_weight* w, const float* x, const b200dec_norm* ln, int lda, int rows, float* part_max,
                   int32_t* part_idx, float* logits, int32_t* status, int pdl, void* stream) {
  B200_REQUIRE(w && w->w && w->scale && x && ln && ln->w && ln->b && part_max && part_idx && status,
               "head_umma: null pointer");
  B200_REQUIRE(w->kind == B200DEC_W_INT8_UMMA && w->k == D_MODEL && w->n % UM == 0, "head_umma: weight kind %d (%d, %d)",
               w->kind, w->n, w->k);
  B200_REQUIRE(rows >= 1 && rows <= 128 && lda % 4 == 0 && ((uintptr_t)x & 15) == 0, "head_umma: rows %d lda %d", rows,
               lda);
  cudaError_t e = cudaFuncSetAttribute(head_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "head_umma: smem attribute: %s", cudaGetErrorString(e));
  const int np = w->n / UM;
  for (int r0 = 0; r0 < rows; r0 += UN) {  // 64 rows per pass (the weights stream once per pass)
    HeadArgs a{};
    a.w = (const uint8_t*)w->w, a.scale = w->scale, a.bias = w->bias, a.x = x + (size_t)r0 * lda;
    a.ln_w = ln->w, a.ln_b = ln->b, a.ln_eps = ln->eps;
    a.part_max = part_max + (size_t)r0 * np, a.part_idx = part_idx + (size_t)r0 * np;
    a.logits = logits ? logits + (size_t)r0 * w->n : nullptr;
    a.status = status, a.lda = lda, a.rows = rows - r0 < UN ? rows - r0 : UN, a.N = w->n;
    e = launch_kernel(head_umma_kernel, dim3(np), dim3(NTHREADS), SMEM_BYTES, (cudaStream_t)stream, 0, pdl, a);
    if (e != cudaSuccess) return fail(B200DEC_ECUDA, "head_umma launch: %s", cudaGetErrorString(e));
  }
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

int b200dec_head_umma(const b200dec_weight* w, const float* x, const b200dec_norm* ln, int lda, int rows,
                      float* part_max, int32_t* part_idx, float* logits, int32_t* status, int pdl, void* stream) {
  return head_umma_impl(w, x, ln, lda, rows, part_max, part_idx, logits, status, pdl, stream);
}

}  // extern "C"
