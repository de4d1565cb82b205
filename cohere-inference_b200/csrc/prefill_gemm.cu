// Cross-attention prefill on the fifth-generation tensor cores: for the packed encoder frames of newly admitted
// requests,  h = frames W_proj^T + b_proj  and  kv = h W_cross^T + b_cross  for all layers at once, with the second
// product written straight into the slot caches (bf16, or int8 with one scale per head vector). There is no fp32
// (frames x 16384) intermediate and no library GEMM.
//
// One kernel computes C(M, N) = A(M, K) B(N, K)^T + bias with fp32 activations A and bf16 weights B:
//   * A is split into two bf16 halves, A = Ah + Al (about 16 bits of mantissa), and the product is Ah B^T + Al B^T,
//     i.e. one bf16 GEMM over K' = 2 K whose second half re-reads the same weights. Both operands are stored in global
//     memory as the exact shared-memory image of their tiles (K-major rows of 128 bytes with the 128-byte swizzle,
//     16 KB per 128-row block of A, 32 KB per 256-channel block of B), so a pipeline stage is two plain
//     cp.async.bulk copies that complete on an mbarrier; nothing else touches the operands.
//   * persistent CTAs, one per SM, walk the (n tile, m tile) list; warp 0 feeds a 4-stage ring, warp 1 issues
//     tcgen05.mma (M 128, N 256, K 16; 4 per stage) into one of two 256-column accumulators in tensor memory and
//     commits stage releases and tile completion to mbarriers, warps 2-5 drain the other accumulator with tcgen05.ld
//     (a thread owns one frame = one tensor-memory lane) while the next tile multiplies.
//   * epilogues: (0) the result, split again into bf16 halves, in the operand image of the next product; (1) a head
//     vector of D consecutive channels = 128 / 256 contiguous bytes of the bf16 cache row of (layer, slot, head,
//     frame); (2) the same quantised as the reference's dec_scatter_kv_q8 does (bf16-round, absmax / 127, rint). The
//     frame's slot and index come from a table of pieces (first row, frames, slot) by binary search.
// Every mbarrier wait is bounded; a wait that runs out sets B200DEC_ST_TIMEOUT, the roles fall through, copies in
// flight are awaited (bounded) and tensor memory is released.
#include "common.cuh"

using namespace b200dec_detail;

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_STAGE = BM * BK * 2, B_STAGE = BN * BK * 2, STAGE_BYTES = A_STAGE + B_STAGE;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;  // slack to align the base to a swizzle atom
constexpr int NTHREADS = 192;                            // producer warp, MMA warp, four epilogue warps
constexpr uint32_t WAIT_LIMIT = 1u << 20;
constexpr int TMEM_COLS = 512;                           // two accumulators of 256 columns

struct GemmArgs {
  const unsigned char* a;  // operand image of the rows: [m tile][2 K / 64][16 KB]
  const unsigned char* w;  // weight image: [n tile][K / 64][32 KB]
  const float* bias;       // (N) or null
  int M, N, K;
  int mode;                // 0 operand image of the next product, 1 bf16 caches, 2 int8 caches
  unsigned char* next;     // mode 0: [m tile][2 N / 64][16 KB]
  const int4* pieces;      // modes 1, 2: (n_pieces) {first row, frames, slot, 0}, first rows ascending from 0
  int n_pieces;
  void* ck;
  void* cv;
  float* cks;
  float* cvs;
  int S1, H, D, T;         // caches (layers, S1, H, T, D)
  int* status;
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
DEVI void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
DEVI void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// K-major tile with the 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart
DEVI uint64_t umma_desc(uint32_t saddr) {
  uint64_t d = (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// bf16 x bf16 -> fp32, both operands K-major, M = 128, N = 256
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
DEVI void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(IDESC), "r"(accumulate)
      : "memory");
}
DEVI void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// 64 consecutive columns of this warp's 32 tensor-memory lanes
DEVI void tmem_ld64(uint32_t taddr, float (&v)[64]) {
  uint32_t d[64];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t* e = d + 32 * h;
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(e[0]), "=r"(e[1]), "=r"(e[2]), "=r"(e[3]), "=r"(e[4]), "=r"(e[5]), "=r"(e[6]), "=r"(e[7]), "=r"(e[8]),
          "=r"(e[9]), "=r"(e[10]), "=r"(e[11]), "=r"(e[12]), "=r"(e[13]), "=r"(e[14]), "=r"(e[15]), "=r"(e[16]),
          "=r"(e[17]), "=r"(e[18]), "=r"(e[19]), "=r"(e[20]), "=r"(e[21]), "=r"(e[22]), "=r"(e[23]), "=r"(e[24]),
          "=r"(e[25]), "=r"(e[26]), "=r"(e[27]), "=r"(e[28]), "=r"(e[29]), "=r"(e[30]), "=r"(e[31])
        : "r"(taddr + 32 * h)
        : "memory");
  }
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(d[i]);
}

// byte offset of (row r, 16-byte chunk c) inside a K-major block of 128-byte rows with the 128-byte swizzle
DEVI int swz(int r, int c) { return (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4); }

// v[0..63] + bias -> the two bf16 halves, as one 128-byte row each of the next product's operand image
DEVI void store_operand_row(const float (&v)[64], unsigned char* hi_blk, unsigned char* lo_blk, int r) {
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint32_t h[4], l[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = v[8 * c + 2 * j], b = v[8 * c + 2 * j + 1];
      h[j] = pack_bf16(a, b);
      l[j] = pack_bf16(a - bf16_lo(h[j]), b - bf16_hi(h[j]));
    }
    *reinterpret_cast<uint4*>(hi_blk + swz(r, c)) = make_uint4(h[0], h[1], h[2], h[3]);
    *reinterpret_cast<uint4*>(lo_blk + swz(r, c)) = make_uint4(l[0], l[1], l[2], l[3]);
  }
}

// the reference's int8 cache format for 64 values already rounded to bf16, given the vector's absmax
DEVI void store_q8_64(const float (&f)[64], float mx, int8_t* dst) {
  const float sc = mx > 0.f ? __fdiv_rn(mx, 127.f) : 1.f, inv = __fdiv_rn(1.f, sc);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int q = __float2int_rn(fminf(fmaxf(__fmul_rn(f[16 * c + i], inv), -127.f), 127.f));
      w[i >> 2] |= (uint32_t)(q & 0xff) << ((i & 3) * 8);
    }
    *reinterpret_cast<uint4*>(dst + 16 * c) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

__global__ void __launch_bounds__(NTHREADS, 1) prefill_gemm_kernel(const GemmArgs p) {
  extern __shared__ unsigned char dyn_smem[];
  unsigned char* smem = dyn_smem + ((1024 - (smem_u32(dyn_smem) & 1023)) & 1023);
  __shared__ __align__(8) uint64_t full[STAGES], empty[STAGES], tfull[2], tempty[2];
  __shared__ uint32_t tmem_base;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int MT = (p.M + BM - 1) / BM, NT = p.N / BN, NKB = p.K / BK, NKB2 = 2 * NKB;
  const int tiles = MT * NT;

  if (tid == 0) {
    for (int i = 0; i < STAGES; ++i) mbar_init(&full[i], 1), mbar_init(&empty[i], 1);
    for (int i = 0; i < 2; ++i) mbar_init(&tfull[i], 1), mbar_init(&tempty[i], 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base)),
                 "n"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = tmem_base;

  if (warp == 0) {
    // ---- producer: two bulk copies per stage --------------------------------------------------------------------------
    if (lane == 0) {
      bool ok = true;
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int mt = tile % MT, nt = tile / MT;
        for (int kb = 0; kb < NKB2; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1);
          if (!ok) break;
          unsigned char* st = smem + s * STAGE_BYTES;
          mbar_expect_tx(&full[s], STAGE_BYTES);
          bulk_load(st, p.a + ((size_t)mt * NKB2 + kb) * A_STAGE, A_STAGE, &full[s]);
          bulk_load(st + A_STAGE, p.w + ((size_t)nt * NKB + kb % NKB) * B_STAGE, B_STAGE, &full[s]);
        }
      }
      if (!ok) {
        atomicOr(p.status, B200DEC_ST_TIMEOUT);
        // the copies already issued must land before this CTA's shared memory is given away
        const uint32_t issued = it < (uint32_t)STAGES ? it : (uint32_t)STAGES;
        for (uint32_t i = 0; i < issued; ++i) {
          const uint32_t jt = it - 1 - i;
          mbar_wait(&full[jt % STAGES], (jt / STAGES) & 1);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issue: one lane ---------------------------------------------------------------------------------------------
    if (lane == 0) {
      bool ok = true;
      uint32_t it = 0, tc = 0;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++tc) {
        const uint32_t buf = tc & 1;
        ok = mbar_wait(&tempty[buf], ((tc >> 1) & 1) ^ 1);  // the epilogue has drained this accumulator
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc = tmem_d + buf * BN;
        for (int kb = 0; kb < NKB2; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(&full[s], (it / STAGES) & 1);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a0 = smem_u32(smem + s * STAGE_BYTES), b0 = a0 + A_STAGE;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) umma_bf16(acc, umma_desc(a0 + k * 32), umma_desc(b0 + k * 32), (kb | k) != 0);
          umma_commit(&empty[s]);  // the stage is free once these MMAs have read it
        }
        if (ok) umma_commit(&tfull[buf]);
      }
      if (!ok) atomicOr(p.status, B200DEC_ST_TIMEOUT);
    }
  } else {
    // ---- epilogue: warp w reads tensor-memory lanes 32 (w % 4) .. + 31; a thread = one row of the tile --------------------
    const int q = warp & 3, row = q * 32 + lane;
    bool ok = true;
    uint32_t tc = 0;
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++tc) {
      const int mt = tile % MT, nt = tile / MT;
      const uint32_t buf = tc & 1;
      ok = mbar_wait(&tfull[buf], (tc >> 1) & 1);
      if (!ok) break;
      tc_fence_after();
      const uint32_t acc = tmem_d + buf * BN + ((uint32_t)(q * 32) << 16);
      const int m = mt * BM + row;
      int slot = -1, frame = 0;
      if (p.mode != 0 && m < p.M) {  // the piece that holds row m: the last one that starts at or before it
        int lo = 0, hi = p.n_pieces - 1;
        while (lo < hi) {
          const int mid = (lo + hi + 1) >> 1;
          if (__ldg(&p.pieces[mid].x) <= m) lo = mid;
          else hi = mid - 1;
        }
        const int4 pc = __ldg(&p.pieces[lo]);
        frame = m - pc.x;
        if (frame >= 0 && frame < pc.y && frame < p.T && pc.z >= 0 && pc.z < p.S1) slot = pc.z;
      }
      for (int c0 = 0; c0 < BN; c0 += 64) {  // warp-uniform trip count: the tensor-memory loads are collective
        const int n0 = nt * BN + c0;
        float v[64];
        tmem_ld64(acc + c0, v);
        if (p.bias) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float4 b = __ldg(reinterpret_cast<const float4*>(p.bias + n0) + i);
            v[4 * i] += b.x, v[4 * i + 1] += b.y, v[4 * i + 2] += b.z, v[4 * i + 3] += b.w;
          }
        }
        if (p.mode == 0) {
          const size_t blk = (size_t)mt * (2 * (p.N / BK)) + n0 / BK;
          store_operand_row(v, p.next + blk * A_STAGE, p.next + (blk + p.N / BK) * A_STAGE, row);
          continue;
        }
        // channel n0 = ((layer * 2 + k|v) * H + head) * D + d
        const int hd = p.H * p.D, l = n0 / (2 * hd), kvi = (n0 / hd) & 1, h = (n0 % hd) / p.D, d0 = n0 % p.D;
        const size_t vec = slot < 0 ? 0 : ((((size_t)l * p.S1 + slot) * p.H + h) * p.T + frame);
        if (p.mode == 1) {
          if (slot >= 0) {
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(kvi ? p.cv : p.ck) + vec * p.D + d0;
#pragma unroll
            for (int c = 0; c < 8; ++c)
              *reinterpret_cast<uint4*>(dst + 8 * c) =
                  make_uint4(pack_bf16(v[8 * c], v[8 * c + 1]), pack_bf16(v[8 * c + 2], v[8 * c + 3]),
                             pack_bf16(v[8 * c + 4], v[8 * c + 5]), pack_bf16(v[8 * c + 6], v[8 * c + 7]));
          }
        } else {
          // int8: the vector's absmax over its D = 64 or 128 channels after rounding to bf16
          float mx = 0.f;
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            v[i] = __bfloat162float(__float2bfloat16_rn(v[i]));
            mx = fmaxf(mx, fabsf(v[i]));
          }
          int8_t* dst = reinterpret_cast<int8_t*>(kvi ? p.cv : p.ck) + vec * p.D + d0;
          if (p.D == 64) {
            if (slot >= 0) {
              store_q8_64(v, mx, dst);
              (kvi ? p.cvs : p.cks)[vec] = mx > 0.f ? __fdiv_rn(mx, 127.f) : 1.f;
            }
          } else {
            // D = 128: this chunk is the first half of its vector (c0 % 128 == 0); fetch the second, then both go out
            float u[64];
            tmem_ld64(acc + c0 + 64, u);
#pragma unroll
            for (int i = 0; i < 64; ++i) {
              const float b = p.bias ? __ldg(p.bias + n0 + 64 + i) : 0.f;
              u[i] = __bfloat162float(__float2bfloat16_rn(u[i] + b));
              mx = fmaxf(mx, fabsf(u[i]));
            }
            if (slot >= 0) {
              store_q8_64(v, mx, dst);
              store_q8_64(u, mx, dst + 64);
              (kvi ? p.cvs : p.cks)[vec] = mx > 0.f ? __fdiv_rn(mx, 127.f) : 1.f;
            }
            c0 += 64;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[buf]);
    }
    if (!ok && lane == 0) atomicOr(p.status, B200DEC_ST_TIMEOUT);
  }
  // ---- release the tensor memory: after every warp is done with it ------------------------------------------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "n"(TMEM_COLS) : "memory");
  }
}

// fp32 rows (m, k) -> the operand image [ceil(m / 128)][2 k / 64][128 rows x 128 B, swizzled]: high halves in the first
// k / 64 blocks of a row tile, low halves in the last; rows past m are zero. One thread per 8 values.
__global__ void pack_rows_kernel(const float* __restrict__ x, int m, int k, int ldx, unsigned char* __restrict__ out) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int cpr = k / 8, mp = (m + BM - 1) / BM * BM;
  if (i >= (size_t)mp * cpr) return;
  const int r = (int)(i / cpr), c = (int)(i % cpr), kb = c >> 3, chunk = c & 7;
  uint32_t h[4] = {0, 0, 0, 0}, l[4] = {0, 0, 0, 0};
  if (r < m) {
    const float4 a = *reinterpret_cast<const float4*>(x + (size_t)r * ldx + c * 8);
    const float4 b = *reinterpret_cast<const float4*>(x + (size_t)r * ldx + c * 8 + 4);
    const float f[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      h[j] = pack_bf16(f[2 * j], f[2 * j + 1]);
      l[j] = pack_bf16(f[2 * j] - bf16_lo(h[j]), f[2 * j + 1] - bf16_hi(h[j]));
    }
  }
  const int nkb = k / BK;
  unsigned char* tile = out + (size_t)(r / BM) * (2 * nkb) * A_STAGE;
  *reinterpret_cast<uint4*>(tile + (size_t)kb * A_STAGE + swz(r % BM, chunk)) = make_uint4(h[0], h[1], h[2], h[3]);
  *reinterpret_cast<uint4*>(tile + (size_t)(nkb + kb) * A_STAGE + swz(r % BM, chunk)) = make_uint4(l[0], l[1], l[2], l[3]);
}

// bf16 weights (n, k) row-major -> the weight image [n / 256][k / 64][256 rows x 128 B, swizzled]; one thread per 16 B
__global__ void tile_weight_kernel(const uint4* __restrict__ w, int n, int k, unsigned char* __restrict__ out) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int cpr = k / 8;
  if (i >= (size_t)n * cpr) return;
  const int r = (int)(i / cpr), c = (int)(i % cpr), kb = c >> 3, chunk = c & 7;
  *reinterpret_cast<uint4*>(out + ((size_t)(r / BN) * (k / BK) + kb) * B_STAGE + swz(r % BN, chunk)) = w[i];
}

}  // namespace

extern "C" {

int64_t b200dec_prefill_rows_bytes(int m, int k) {
  if (m < 0 || k <= 0 || k % BK) return -1;
  return (int64_t)((m + BM - 1) / BM) * BM * 2 * k * 2;
}

int b200dec_prefill_pack_rows(const float* x, int m, int k, int ldx, void* image, void* stream) {
  B200_REQUIRE(x && image && m >= 1 && k >= BK && k % BK == 0 && ldx >= k && ldx % 4 == 0 && ((uintptr_t)x & 15) == 0 &&
                   ((uintptr_t)image & 1023) == 0, "prefill_pack_rows: m %d k %d ldx %d (k a multiple of 64, image 1 KB aligned)",
               m, k, ldx);
  const size_t total = (size_t)((m + BM - 1) / BM) * BM * (k / 8);
  pack_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, m, k, ldx, (unsigned char*)image);
  return check_launch("prefill_pack_rows");
}

int b200dec_prefill_tile_weight(const void* w_bf16, int n, int k, void* image, void* stream) {
  B200_REQUIRE(w_bf16 && image && n >= BN && n % BN == 0 && k >= BK && k % BK == 0 && ((uintptr_t)w_bf16 & 15) == 0 &&
                   ((uintptr_t)image & 1023) == 0, "prefill_tile_weight: (%d, %d) must be multiples of (256, 64)", n, k);
  const size_t total = (size_t)n * (k / 8);
  tile_weight_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const uint4*)w_bf16, n, k,
                                                                                        (unsigned char*)image);
  return check_launch("prefill_tile_weight");
}

int b200dec_prefill_gemm(const void* rows_image, int m, int k, const void* weight_image, const float* bias, int n,
                         int mode, void* next_image, const int32_t* pieces, int n_pieces, void* ck, void* cv,
                         float* ck_scale, float* cv_scale, int layers, int slots_plus_1, int heads, int head_dim,
                         int frames, int32_t* status, void* stream) {
  B200_REQUIRE(rows_image && weight_image && status, "prefill_gemm: null pointer");
  B200_REQUIRE(m >= 1 && k >= BK && k % BK == 0 && n >= BN && n % BN == 0, "prefill_gemm: m %d k %d n %d", m, k, n);
  B200_REQUIRE(((uintptr_t)rows_image & 1023) == 0 && ((uintptr_t)weight_image & 1023) == 0 && ((uintptr_t)bias & 15) == 0,
               "prefill_gemm: the operand images must be 1 KB aligned, the bias 16-byte aligned");
  B200_REQUIRE(mode >= 0 && mode <= 2, "prefill_gemm: mode %d", mode);
  if (mode == 0) {
    B200_REQUIRE(next_image && ((uintptr_t)next_image & 1023) == 0, "prefill_gemm: mode 0 writes the next operand image");
  } else {
    B200_REQUIRE(pieces && n_pieces >= 1 && ck && cv && ((uintptr_t)pieces & 15) == 0 && ((uintptr_t)ck & 15) == 0 &&
                     ((uintptr_t)cv & 15) == 0, "prefill_gemm: the cache modes need the piece table and the caches");
    B200_REQUIRE((head_dim == 64 || head_dim == 128) && layers >= 1 && heads >= 1 &&
                     n == layers * 2 * heads * head_dim, "prefill_gemm: n %d != layers %d x 2 x heads %d x head_dim %d", n,
                 layers, heads, head_dim);
    B200_REQUIRE(mode != 2 || (ck_scale && cv_scale), "prefill_gemm: int8 caches need their scales");
  }
  cudaError_t e = cudaFuncSetAttribute(prefill_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "prefill_gemm: smem attribute: %s", cudaGetErrorString(e));
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int tiles = ((m + BM - 1) / BM) * (n / BN);
  GemmArgs a{(const unsigned char*)rows_image, (const unsigned char*)weight_image, bias, m, n, k, mode,
             (unsigned char*)next_image, (const int4*)pieces, n_pieces, ck, cv, ck_scale, cv_scale, slots_plus_1, heads,
             head_dim, frames, status};
  e = launch_kernel(prefill_gemm_kernel, dim3(tiles < sms ? tiles : sms), dim3(NTHREADS), SMEM_BYTES,
                    (cudaStream_t)stream, 0, false, a);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "prefill_gemm launch: %s", cudaGetErrorString(e));
  return 0;
}

}  // extern "C"
