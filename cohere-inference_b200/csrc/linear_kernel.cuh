// Small-M projection kernel: out (rows, N) = act(A (rows, K) x W^T * scale + bias), rows <= 128. See linear.cu for
// the design notes and the tiled weight layouts; this header holds the kernel template and its launcher so that each
// weight kind compiles in its own translation unit.
#pragma once
#include <cooperative_groups.h>

#include "common.cuh"

namespace b200dec_detail {

namespace cg = cooperative_groups;

struct LinArgs {
  const uint8_t* w;
  const uint32_t* meta;
  const float* scale;
  const float* bias;
  const void* a;
  const float* ln_w;     // LayerNorm folded in (a = fp32 residual stream) when non-null: gamma ...
  const float* ln_g;     // ... g[n] = sum_k gamma[k] W[n][k] ...
  const float* ln_bias;  // ... and sum_k beta[k] W[n][k], both of the dequantised weights
  void* out;
  // Link to the LayerNorm-folding projection that reads the rows an OUT_F32_ADD call updates (all null: none): the
  // rows times that LayerNorm's gamma as fp16 (its operand), and per finishing CTA the rows' sum and sum of squares
  // over its channels, stats_out (rows, gridDim.y * KSPLIT, 2).
  const float* next_gamma;
  __half* out16;
  float* stats_out;
  // The reading side (LN == 2): those partial sums, (rows, stats_slots, 2).
  const float* stats_in;
  int stats_slots;
  float* part_max;
  int* part_idx;
  float* logits;
  float ln_eps;
  int lda, ldo, rows, N, out_kind, act, head;
  KvPrefetch pf;  // keys and values of the next attention launch to start on their way into L2 (sched null: none)
  int* status;    // or null: receives B200DEC_ST_TIMEOUT if the bounded wait for the cluster's partial results runs out
};

template <int WT>
struct WTraits;
template <>
struct WTraits<B200DEC_W_INT8> {
  static constexpr int KPB = 64, STEPS = 4, PAD = 16;
};
template <>
struct WTraits<B200DEC_W_BF16> {
  static constexpr int KPB = 32, STEPS = 2, PAD = 64;
};
template <>
struct WTraits<B200DEC_W_F16> {  // the layout of B200DEC_W_BF16, the arithmetic of the int8 kinds
  static constexpr int KPB = 32, STEPS = 2, PAD = 64;
};
template <>
struct WTraits<B200DEC_W_INT8_24> {
  static constexpr int KPB = 128, STEPS = 8, PAD = 64;
};

DEVI void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
DEVI void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 4 offset-binary bytes (q + 128, k .. k+3) -> half2(q0, q1), half2(q2, q3); exact: 0x64uu is the half 1024 + uu
DEVI void widen_u8(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t x0 = __byte_perm(w, 0x64646464u, 0x4140);
  const uint32_t x1 = __byte_perm(w, 0x64646464u, 0x4342);
  const __half2 magic = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));  // 1152
  const __half2 r0 = __hsub2(*reinterpret_cast<const __half2*>(&x0), magic);
  const __half2 r1 = __hsub2(*reinterpret_cast<const __half2*>(&x1), magic);
  lo = *reinterpret_cast<const uint32_t*>(&r0);
  hi = *reinterpret_cast<const uint32_t*>(&r1);
}

DEVI float act_fn(float v, int act) {
  if (act == B200DEC_ACT_RELU) return fmaxf(v, 0.f);
  if (act == B200DEC_ACT_GELU) return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
  return v;
}

// 4 fp32 activations -> their 16-bit operand: the nearest half / bf16 and, when split, the rounded remainder
template <bool BF, bool SPLIT>
DEVI void to_operand(float4 v, uint2& hi, uint2& lo) {
  if constexpr (BF) {
    hi = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
    if constexpr (SPLIT)
      lo = make_uint2(pack_bf16(v.x - bf16_lo(hi.x), v.y - bf16_hi(hi.x)),
                      pack_bf16(v.z - bf16_lo(hi.y), v.w - bf16_hi(hi.y)));
  } else {
    const float c0 = clamp_h(v.x), c1 = clamp_h(v.y), c2 = clamp_h(v.z), c3 = clamp_h(v.w);
    const __half2 h01 = __floats2half2_rn(c0, c1), h23 = __floats2half2_rn(c2, c3);
    hi = make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
    if constexpr (SPLIT) {
      const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
      lo = make_uint2(pack_f16(c0 - f01.x, c1 - f01.y), pack_f16(c2 - f23.x, c3 - f23.y));
    }
  }
}

template <int WT, bool SPLIT, int LN, int NW, int KSLICE, int KSPLIT, int MB>
struct LinSmem {
  static constexpr int RS = KSLICE * 2 + WTraits<WT>::PAD;  // bytes per staged activation row
  static constexpr int BN = NW * 16;
  static constexpr int A_BYTES = MB * RS * (SPLIT ? 2 : 1);
  static constexpr int RECV_BYTES = MB * BN * 4;       // [KSPLIT][MB][BN / KSPLIT] partial sums pushed by the cluster
  // fp32 source rows are first copied asynchronously into shared memory (slices up to 256 wide; wider ones are
  // converted straight from registers)
  static constexpr bool RAW_STAGE = (LN == 1 || SPLIT) && KSLICE <= 256;
  static constexpr int RAW_BYTES = RAW_STAGE ? MB * KSLICE * 4 : 0;
  static constexpr int STATS_BYTES = LN == 1 ? KSPLIT * MB * 8 : LN == 2 ? MB * 8 : 0;  // per slice / totals  // [KSPLIT][MB] (sum, sum of squares) of each slice
  static constexpr int OFF_A = 0, OFF_RECV = OFF_A + A_BYTES, OFF_RAW = OFF_RECV + RECV_BYTES,
                       OFF_STATS = OFF_RAW + RAW_BYTES, TOTAL = OFF_STATS + STATS_BYTES;
};

// WT: weight storage. SPLIT: the activation operand is two 16-bit halves (hi + lo) of an fp32 value, else one fp16.
// LN: the operand is LayerNorm(a) of the fp32 rows a with the normalisation folded into the epilogue: with a per-row
// shift c (the mean of the row's first four values) the kernel multiplies (a - c) * gamma, every CTA also sums its
// slice's (a - c) and (a - c)^2, and the finishing CTA applies  y = rstd * (acc * scale - (mean - c) * g) + bias',
// which equals LayerNorm(a) W^T + bias exactly (g and bias' are precomputed per output channel). NW warps = 16 NW
// channels per CTA; KSLICE k-values per CTA, KSPLIT CTAs per cluster (K = KSLICE * KSPLIT); MB: row capacity.
// CTAs per SM the register allocation must leave room for. The 2:4 fc2 at 65-128 rows is dealt as 8 x 16 x 4 = 512
// CTAs of 32 rows: they only run as one wave with four per SM, i.e. at no more than 128 registers (the compiler sits at
// 128-129 for that tile; the one register more cost a second wave, +3 us per launch, 5 % of a 128-row step). The dense
// int8 tile of the same shape also serves fc2 at 33-64 rows (two CTAs of 32 rows per tile, one wave either way), where
// holding it to 128 registers instead of its 140 measured 1.3 us slower per launch: it keeps its registers.
template <int WT, int NW, int KSLICE, int MB>
constexpr int linear_min_ctas() {
  return (WT == B200DEC_W_INT8_24 && NW == 4 && KSLICE == 512 && MB == 32) ? 4 : 1;
}

template <int WT, bool SPLIT, int LN, int NW, int KSLICE, int KSPLIT, int MB>
__global__ void __launch_bounds__(NW * 32, linear_min_ctas<WT, NW, KSLICE, MB>()) linear_kernel(const LinArgs p_in) {
  // How the cluster's partial results travel. st.async onto an mbarrier of the owning CTA pays while a CTA is owed few
  // values (each one also updates that mbarrier): measured at rows x 16 NW = 2048 values per CTA -0.2 to -0.4 us per
  // launch against stores + a cluster barrier, at 16384 (the 2:4 fc1 at 128 rows) +1.2 us. The choice is a property
  // of the tile, so only one of the two paths is compiled into a kernel.
  constexpr bool ASYNC_X = MB * NW <= 256;
  __shared__ __align__(8) uint64_t xbar;  // counts the bytes this CTA is owed by its cluster (ASYNC_X)
  if (ASYNC_X && threadIdx.x == 0) xbar_init(&xbar);
  cluster_arrive_entry();  // completed by cluster_wait_entry() before this CTA's first remote store
  LinArgs p = p_in;
  if (gridDim.z > 1) {  // the rows are dealt over blockIdx.z, MB each (fp16 operands only)
    const int row0 = blockIdx.z * MB;
    p.a = reinterpret_cast<const char*>(p.a) + (size_t)row0 * p.lda * 2;
    p.out = reinterpret_cast<char*>(p.out) + (size_t)row0 * p.ldo * (p.out_kind == B200DEC_OUT_F16 ? 2 : 4);
    if (p.out16) p.out16 += (size_t)row0 * p.ldo;
    if (p.stats_out) p.stats_out += (size_t)row0 * (gridDim.y * KSPLIT) * 2;
    if (p.stats_in) p.stats_in += (size_t)row0 * p.stats_slots * 2;
    p.rows = p.rows - row0 < MB ? p.rows - row0 : MB;
  }
  using T = WTraits<WT>;
  using S = LinSmem<WT, SPLIT, LN, NW, KSLICE, KSPLIT, MB>;
  constexpr int KPB = T::KPB, STEPS = T::STEPS, NBLK = KSLICE / KPB, NT = NW * 32, BN = NW * 16, K = KSLICE * KSPLIT;
  constexpr int RS = S::RS, CPR = BN / KSPLIT, GPR = CPR / 4, NB = MB / 8, NBG = NB < 8 ? NB : 8;
  constexpr bool BF = WT == B200DEC_W_BF16, W16 = BF || WT == B200DEC_W_F16;  // bf16 arithmetic; 16-bit weight layout
  constexpr bool F32SRC = LN == 1 || SPLIT;  // the source rows are fp32
  static_assert(LN != 2 || (!SPLIT && KSLICE <= 256), "fp16 source rows: one fp16 operand, a row's chunks within a warp");
  static_assert(CPR % 8 == 0, "each CTA finishes a multiple of 8 channels");
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint32_t lut[32];
  unsigned char* a_hi = smem + S::OFF_A;
  unsigned char* a_lo = a_hi + MB * RS;
  float* recv = reinterpret_cast<float*>(smem + S::OFF_RECV);
  float* raw = reinterpret_cast<float*>(smem + S::OFF_RAW);  // the async copy of the fp32 rows (RAW_STAGE)
  float2* stats = reinterpret_cast<float2*>(smem + S::OFF_STATS);

  cg::cluster_group cluster = cg::this_cluster();
  const int rank = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int nt16 = blockIdx.y * NW + warp;  // this warp's 16 channels
  const int k0 = rank * KSLICE;
  // ---- prologue: the warp's whole weight slice into registers (independent of the previous kernel) -------------
  uint4 wr[NBLK][2];
  uint32_t mr[WT == B200DEC_W_INT8_24 ? NBLK : 1][2];
  {
    const size_t blk0 = (size_t)nt16 * (K / KPB) + k0 / KPB;
    const uint8_t* wp = p.w + blk0 * 1024 + lane * 16;
#pragma unroll
    for (int b = 0; b < NBLK; ++b) {
      wr[b][0] = ld_stream16(wp + (size_t)b * 1024);
      wr[b][1] = ld_stream16(wp + (size_t)b * 1024 + 512);
    }
    if constexpr (WT == B200DEC_W_INT8_24) {
      const uint32_t* mp = p.meta + blk0 * 64 + lane;
#pragma unroll
      for (int b = 0; b < NBLK; ++b) {
        mr[b][0] = ld_stream4(mp + (size_t)b * 64);
        mr[b][1] = ld_stream4(mp + (size_t)b * 64 + 32);
      }
      // byte-permute controls: dense byte q of a group takes kept byte 0/1 (even step) or 2/3 (odd step) of the
      // register when q is the first / second kept position, else the zero byte (index 4 = 0x80)
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
  }
  pdl_wait();
  pdl_trigger();  // at once: the dependent's CTAs need ~2 us to start and fetch their weights, more than is left of this one
  if (ASYNC_X && tid == 0)  // partial tiles from every CTA of the cluster (this one included) and the rows' sums
    xbar_expect(&xbar, (uint32_t)(KSPLIT * p.rows * CPR * 4 + (LN == 2 ? p.rows * 8 : LN == 1 ? KSPLIT * p.rows * 8 : 0)));
  if (p.pf.sched)
    kv_prefetch_issue(p.pf, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x,
                      gridDim.x * gridDim.y * gridDim.z, tid, NT);

  // ---- stage the activations of this K slice ---------------------------------------------------------------------
  const int ntiles = (p.rows + 7) >> 3, rows8 = ntiles * 8;
  if constexpr (!F32SRC) {
    constexpr int CH = KSLICE / 8;  // 16-byte chunks per row
    const __half* A = reinterpret_cast<const __half*>(p.a);
    for (int i = tid; i < rows8 * CH; i += NT) {
      const int r = i / CH, c = i % CH;
      if (r < p.rows)
        cp_async16(a_hi + r * RS + c * 16, A + (size_t)r * p.lda + k0 + c * 8);
      else
        *reinterpret_cast<uint4*>(a_hi + r * RS + c * 16) = make_uint4(0, 0, 0, 0);
    }
    if constexpr (LN == 2) {
      // The rows are already this projection's operand (x * gamma as fp16, written by the projection that updated x):
      // nothing to convert. Their statistics come as one partial (sum, sum of squares) per row and finishing CTA of
      // that projection; the cluster shares the adding up: this CTA takes rows rank, rank + KSPLIT, ... (a warp per
      // row, lanes over the partials, fixed order) and hands each total to every CTA of the cluster.
      constexpr int RPW = (MB + KSPLIT * NW - 1) / (KSPLIT * NW);  // rows per warp, all their loads issued at once
      float2 v[RPW][4];                                              // up to 128 partials per row: 4 per lane
#pragma unroll
      for (int j = 0; j < RPW; ++j) {
        const int r = rank + KSPLIT * (warp + NW * j);
        const float2* part = reinterpret_cast<const float2*>(p.stats_in) + (size_t)r * p.stats_slots;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          v[j][i] = (r < p.rows && lane + 32 * i < p.stats_slots) ? __ldcg(part + lane + 32 * i) : make_float2(0.f, 0.f);
      }
      cluster_wait_entry();
#pragma unroll
      for (int j = 0; j < RPW; ++j) {
        const int r = rank + KSPLIT * (warp + NW * j);
        float s1 = (v[j][0].x + v[j][1].x) + (v[j][2].x + v[j][3].x), s2 = (v[j][0].y + v[j][1].y) + (v[j][2].y + v[j][3].y);
        s1 = warp_sum(s1), s2 = warp_sum(s2);
        if (r < p.rows && lane < KSPLIT) {
          if constexpr (ASYNC_X)
            st_async_f32x2(map_to_rank(smem_addr_u32(stats + r), lane), make_float2(s1, s2),
                           map_to_rank(smem_addr_u32(&xbar), lane));
          else
            cluster.map_shared_rank(stats, lane)[r] = make_float2(s1, s2);
        }
      }
    }
    cp_async_wait_all();

  } else {
    // fp32 rows: 8 lanes per row, each with KSLICE / 32 independent 16-byte loads in flight; converted (and, for the
    // folded LayerNorm, shifted, scaled by gamma and summed) on the way to shared memory
    constexpr int J = KSLICE / 32;
    constexpr int RPG = (MB + NT / 8 - 1) / (NT / 8);  // rows per 8-lane group
    const float* A = reinterpret_cast<const float*>(p.a);
    const int l8 = tid & 7;
    float shift[RPG];
    if constexpr (S::RAW_STAGE) {
      constexpr int CH = KSLICE / 4;
      for (int i = tid; i < p.rows * CH; i += NT) {
        const int r = i / CH, c = i % CH;
        cp_async16(raw + r * KSLICE + c * 4, A + (size_t)r * p.lda + k0 + c * 4);
      }
    }
    if constexpr (LN) {  // the rows' shifts, fetched while the copies are in flight
#pragma unroll
      for (int it = 0; it < RPG; ++it) {
        const int r = (tid >> 3) + it * (NT / 8);
        shift[it] = 0.f;
        if (r < p.rows) {
          const float4 f = ld_cg_f4(A + (size_t)r * p.lda);
          shift[it] = 0.25f * (f.x + f.y + f.z + f.w);
        }
      }
    }
    float4 gam[LN ? J : 1];  // this lane's gammas, the same for every row
    if constexpr (LN) {
#pragma unroll
      for (int j = 0; j < J; ++j) gam[j] = __ldg(reinterpret_cast<const float4*>(p.ln_w + k0 + (j * 8 + l8) * 4));
    }
    if constexpr (S::RAW_STAGE) {
      cp_async_wait_all();
      __syncthreads();
    }
    float s1[RPG], s2[RPG];
#pragma unroll
    for (int it = 0; it < RPG; ++it) {  // no early exit: the iterations are independent and interleave
      const int r = (tid >> 3) + it * (NT / 8);
      const bool live = r < p.rows;
      s1[it] = 0.f, s2[it] = 0.f;
      if (r < rows8) {  // whole warps agree (rows8 % 8 == 0, 4 row groups per warp)
        const float c = LN ? shift[it] : 0.f;
#pragma unroll
        for (int j = 0; j < J; ++j) {
          uint2 hi = make_uint2(0, 0), lo = make_uint2(0, 0);
          if (live) {
            float4 x;
            if constexpr (S::RAW_STAGE) x = *reinterpret_cast<const float4*>(raw + r * KSLICE + (j * 8 + l8) * 4);
            else x = ld_cg_f4(A + (size_t)r * p.lda + k0 + (j * 8 + l8) * 4);
            if constexpr (LN) {
              x.x -= c, x.y -= c, x.z -= c, x.w -= c;
              s1[it] += (x.x + x.y) + (x.z + x.w);
              s2[it] += (x.x * x.x + x.y * x.y) + (x.z * x.z + x.w * x.w);
              x.x *= gam[j].x, x.y *= gam[j].y, x.z *= gam[j].z, x.w *= gam[j].w;
            }
            to_operand<BF, SPLIT>(x, hi, lo);
          }
          *reinterpret_cast<uint2*>(a_hi + r * RS + (j * 8 + l8) * 8) = hi;
          if constexpr (SPLIT) *reinterpret_cast<uint2*>(a_lo + r * RS + (j * 8 + l8) * 8) = lo;
        }
      }
    }
    if constexpr (LN) {
#pragma unroll
      for (int o = 1; o < 8; o <<= 1)
#pragma unroll
        for (int it = 0; it < RPG; ++it) {
          s1[it] += __shfl_xor_sync(0xffffffffu, s1[it], o);
          s2[it] += __shfl_xor_sync(0xffffffffu, s2[it], o);
        }
      cluster_wait_entry();
#pragma unroll
      for (int it = 0; it < RPG; ++it) {
        const int r = (tid >> 3) + it * (NT / 8);
        if (r < p.rows && l8 < KSPLIT) {
          if constexpr (ASYNC_X)
            st_async_f32x2(map_to_rank(smem_addr_u32(stats + rank * MB + r), l8), make_float2(s1[it], s2[it]),
                           map_to_rank(smem_addr_u32(&xbar), l8));
          else
            cluster.map_shared_rank(stats, l8)[rank * MB + r] = make_float2(s1[it], s2[it]);
        }
      }
    }
  }
  __syncthreads();

  // ---- multiply: consecutive MMAs go to different accumulators (up to 8 row tiles in flight) ----------------------
  float acc[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[nb][e] = 0.f;

#pragma unroll
  for (int b = 0; b < NBLK; ++b) {
    uint32_t af[STEPS][4];  // weight fragments of the block's steps
    if constexpr (WT == B200DEC_W_INT8) {
      const uint32_t r0[4] = {wr[b][0].x, wr[b][0].y, wr[b][0].z, wr[b][0].w};
      const uint32_t r1[4] = {wr[b][1].x, wr[b][1].y, wr[b][1].z, wr[b][1].w};
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        widen_u8(r0[s], af[s][0], af[s][2]);
        widen_u8(r1[s], af[s][1], af[s][3]);
      }
    } else if constexpr (W16) {
      af[0][0] = wr[b][0].x, af[0][2] = wr[b][0].y, af[1][0] = wr[b][0].z, af[1][2] = wr[b][0].w;
      af[0][1] = wr[b][1].x, af[0][3] = wr[b][1].y, af[1][1] = wr[b][1].z, af[1][3] = wr[b][1].w;
    } else {
      const uint32_t r0[4] = {wr[b][0].x ^ 0x80808080u, wr[b][0].y ^ 0x80808080u, wr[b][0].z ^ 0x80808080u,
                              wr[b][0].w ^ 0x80808080u};
      const uint32_t r1[4] = {wr[b][1].x ^ 0x80808080u, wr[b][1].y ^ 0x80808080u, wr[b][1].z ^ 0x80808080u,
                              wr[b][1].w ^ 0x80808080u};
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        const uint32_t c0 = lut[((mr[b][0] >> (4 * s)) & 15u) | ((s & 1) << 4)];
        const uint32_t c1 = lut[((mr[b][1] >> (4 * s)) & 15u) | ((s & 1) << 4)];
        widen_u8(__byte_perm(r0[s >> 1], 0x80808080u, c0), af[s][0], af[s][2]);
        widen_u8(__byte_perm(r1[s >> 1], 0x80808080u, c1), af[s][1], af[s][3]);
      }
    }
#pragma unroll
    for (int c = 0; c < STEPS / 2; ++c) {  // one 16-byte chunk of a row = the lane's k-values of two steps
      int col;                             // first k of the chunk inside the slice
      if constexpr (WT == B200DEC_W_INT8) col = b * 64 + t * 16 + c * 8;
      else if constexpr (W16) col = b * 32 + t * 8;
      else col = b * 128 + (4 * c + t) * 8;
#pragma unroll
      for (int n0 = 0; n0 < NB; n0 += NBG) {
        if (n0 < ntiles) {
          uint4 h[NBG], l[SPLIT ? NBG : 1];
#pragma unroll
          for (int i = 0; i < NBG; ++i) {
            h[i] = *reinterpret_cast<const uint4*>(a_hi + ((n0 + i) * 8 + g) * RS + col * 2);
            if constexpr (SPLIT) l[i] = *reinterpret_cast<const uint4*>(a_lo + ((n0 + i) * 8 + g) * RS + col * 2);
          }
#pragma unroll
          for (int e = 0; e < 2; ++e) {
#pragma unroll
            for (int i = 0; i < NBG; ++i) {
              if (n0 + i < ntiles) {
                const uint32_t b0 = e ? h[i].z : h[i].x, b1 = e ? h[i].w : h[i].y;
                if constexpr (BF) mma_bf16(acc[n0 + i], af[2 * c + e], b0, b1);
                else mma_f16(acc[n0 + i], af[2 * c + e], b0, b1);
              }
            }
            if constexpr (SPLIT) {
#pragma unroll
              for (int i = 0; i < NBG; ++i) {
                if (n0 + i < ntiles) {
                  const uint32_t b0 = e ? l[i].z : l[i].x, b1 = e ? l[i].w : l[i].y;
                  if constexpr (BF) mma_bf16(acc[n0 + i], af[2 * c + e], b0, b1);
                  else mma_f16(acc[n0 + i], af[2 * c + e], b0, b1);
                }
              }
            }
          }
        }
      }
    }
  }

  // ---- partial tile -> the CTAs that own its channels (distributed shared memory), one cluster barrier ------------
  // Straight from the accumulators: a warp's store instruction covers 8 consecutive channels (32 bytes) of 4 rows,
  // all owned by one CTA of the cluster.
  if constexpr (LN == 0) cluster_wait_entry();  // with a LayerNorm the statistics were the first remote stores
  {
    const int ch0 = warp * 16 + g, ch1 = ch0 + 8;
    if constexpr (ASYNC_X) {
      const uint32_t d0 = map_to_rank(smem_addr_u32(recv + rank * MB * CPR + ch0 % CPR), ch0 / CPR);
      const uint32_t d1 = map_to_rank(smem_addr_u32(recv + rank * MB * CPR + ch1 % CPR), ch1 / CPR);
      const uint32_t b0 = map_to_rank(smem_addr_u32(&xbar), ch0 / CPR), b1 = map_to_rank(smem_addr_u32(&xbar), ch1 / CPR);
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        if (nb < ntiles) {
          const int r = nb * 8 + 2 * t;
          if (r < p.rows) st_async_f32(d0 + r * CPR * 4, acc[nb][0], b0), st_async_f32(d1 + r * CPR * 4, acc[nb][2], b1);
          if (r + 1 < p.rows)
            st_async_f32(d0 + (r + 1) * CPR * 4, acc[nb][1], b0), st_async_f32(d1 + (r + 1) * CPR * 4, acc[nb][3], b1);
        }
      }
    } else {
      float* dst0 = cluster.map_shared_rank(recv, ch0 / CPR) + rank * MB * CPR + ch0 % CPR;
      float* dst1 = cluster.map_shared_rank(recv, ch1 / CPR) + rank * MB * CPR + ch1 % CPR;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        if (nb < ntiles) {
          const int r = nb * 8 + 2 * t;
          if (r < p.rows) dst0[r * CPR] = acc[nb][0], dst1[r * CPR] = acc[nb][2];
          if (r + 1 < p.rows) dst0[(r + 1) * CPR] = acc[nb][1], dst1[(r + 1) * CPR] = acc[nb][3];
        }
      }
    }
  }
  // this thread's share of the finished tile: row r, channels n .. n+3; the residual it adds to is fetched now so
  // that its latency overlaps the barrier
  const int items = p.rows * GPR;
  const bool one_item = items <= NT;  // the common case: at most one item per thread
  float4 resid = make_float4(0.f, 0.f, 0.f, 0.f);
  if (one_item && tid < items && !p.head && p.out_kind == B200DEC_OUT_F32_ADD)
    resid = __ldcg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.out) + (size_t)(tid / GPR) * p.ldo +
                                                   blockIdx.y * BN + rank * CPR + (tid % GPR) * 4));
  // likewise the per-channel vectors of the epilogue (the same four channels for every item of this thread)
  const int n_mine = blockIdx.y * BN + rank * CPR + (tid % GPR) * 4;
  const float4 one4 = make_float4(1.f, 1.f, 1.f, 1.f), zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  const bool pre = NT % GPR == 0;  // then `it % GPR` is the same for all of a thread's items
  const float4 sc_pre = (pre && p.scale) ? __ldg(reinterpret_cast<const float4*>(p.scale + n_mine)) : one4;
  const float4 bb_pre = (pre && p.bias) ? __ldg(reinterpret_cast<const float4*>(p.bias + n_mine)) : zero4;
  const float4 gn_pre = (pre && p.out16) ? __ldg(reinterpret_cast<const float4*>(p.next_gamma + n_mine)) : one4;
  float4 gg_pre = zero4, lb_pre = zero4;
  if constexpr (LN) {
    if (pre) {
      gg_pre = __ldg(reinterpret_cast<const float4*>(p.ln_g + n_mine));
      lb_pre = __ldg(reinterpret_cast<const float4*>(p.ln_bias + n_mine));
    }
  }
  if constexpr (ASYNC_X) {  // everything this CTA is owed has landed (nobody writes to it afterwards: it may leave)
    if (!xbar_wait(&xbar, 1u << 22) && lane == 0 && p.status) atomicOr(p.status, B200DEC_ST_TIMEOUT);
  } else {
    cluster.sync();  // all partials (and slice statistics) have landed; nobody touches remote shared memory after this
  }

  const int padded = (items + 31) & ~31;
  for (int it = tid; it < padded; it += NT) {
    const bool live = it < items;
    const int r = live ? it / GPR : 0, c4 = live ? it % GPR : 0;
    const int n = blockIdx.y * BN + rank * CPR + c4 * 4;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) {
#pragma unroll
      for (int q = 0; q < KSPLIT; ++q) {  // fixed rank order: the same bits whatever the timing
        const float4 v = *reinterpret_cast<const float4*>(recv + (q * MB + r) * CPR + c4 * 4);
        s.x += v.x, s.y += v.y, s.z += v.z, s.w += v.w;
      }
      if (p.scale) {
        const float4 sc = pre ? sc_pre : *reinterpret_cast<const float4*>(p.scale + n);
        s.x *= sc.x, s.y *= sc.y, s.z *= sc.z, s.w *= sc.w;
      }
      if constexpr (LN) {
        float s1 = 0.f, s2 = 0.f;
        if constexpr (LN == 2) {
          const float2 st = stats[r];
          s1 = st.x, s2 = st.y;
        } else {
#pragma unroll
          for (int q = 0; q < KSPLIT; ++q) {
            const float2 st = stats[q * MB + r];
            s1 += st.x, s2 += st.y;
          }
        }
        const float dm = s1 * (1.f / K);  // mean - shift
        const float rstd = rsqrtf(fmaxf(s2 * (1.f / K) - dm * dm, 0.f) + p.ln_eps);
        const float4 gg = pre ? gg_pre : *reinterpret_cast<const float4*>(p.ln_g + n);
        const float4 lb = pre ? lb_pre : *reinterpret_cast<const float4*>(p.ln_bias + n);
        s.x = rstd * (s.x - dm * gg.x) + lb.x, s.y = rstd * (s.y - dm * gg.y) + lb.y;
        s.z = rstd * (s.z - dm * gg.z) + lb.z, s.w = rstd * (s.w - dm * gg.w) + lb.w;
      }
      if (p.bias) {
        const float4 bb = pre ? bb_pre : *reinterpret_cast<const float4*>(p.bias + n);
        s.x += bb.x, s.y += bb.y, s.z += bb.z, s.w += bb.w;
      }
      s.x = act_fn(s.x, p.act), s.y = act_fn(s.y, p.act), s.z = act_fn(s.z, p.act), s.w = act_fn(s.w, p.act);
      if (!p.head) {
        if (p.out_kind == B200DEC_OUT_F16) {
          *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(p.out) + (size_t)r * p.ldo + n) =
              make_uint2(pack_f16(s.x, s.y), pack_f16(s.z, s.w));
        } else {
          float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + (size_t)r * p.ldo + n);
          if (p.out_kind == B200DEC_OUT_F32_ADD) {
            const float4 x = one_item ? resid : __ldcg(o);
            s.x += x.x, s.y += x.y, s.z += x.z, s.w += x.w;
            if (p.out16) {
              const float4 gn = pre ? gn_pre : *reinterpret_cast<const float4*>(p.next_gamma + n);
              *reinterpret_cast<uint2*>(p.out16 + (size_t)r * p.ldo + n) =
                  make_uint2(pack_f16(s.x * gn.x, s.y * gn.y), pack_f16(s.z * gn.z, s.w * gn.w));
            }
          }
          *o = s;
        }
      } else if (p.logits) {
        *reinterpret_cast<float4*>(p.logits + (size_t)r * p.N + n) = s;
      }
    }
    if (p.stats_out) {  // warp-uniform; the row's GPR consecutive lanes add up their channels, one of them publishes
      float p1 = live ? (s.x + s.y) + (s.z + s.w) : 0.f;
      float p2 = live ? (s.x * s.x + s.y * s.y) + (s.z * s.z + s.w * s.w) : 0.f;
#pragma unroll
      for (int o = 1; o < GPR && o < 32; o <<= 1) {
        p1 += __shfl_xor_sync(0xffffffffu, p1, o);
        p2 += __shfl_xor_sync(0xffffffffu, p2, o);
      }
      if (live && c4 == 0)
        reinterpret_cast<float2*>(p.stats_out)[(size_t)r * (gridDim.y * KSPLIT) + blockIdx.y * KSPLIT + rank] =
            make_float2(p1, p2);
    }
    if (p.head) {
      // first index of the maximum over this CTA's channels of row r (NaN never wins): GPR consecutive lanes
      float best = -INFINITY;
      int arg = 0x7fffffff;
      if (live) {
        const float v[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (v[e] > best) best = v[e], arg = n + e;
      }
#pragma unroll
      for (int o = 1; o < GPR && o < 32; o <<= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ob > best || (ob == best && oa < arg)) best = ob, arg = oa;
      }
      if (live && c4 == 0) {
        const int np = (p.N / BN) * KSPLIT, slot = blockIdx.y * KSPLIT + rank;
        p.part_max[(size_t)r * np + slot] = best;
        p.part_idx[(size_t)r * np + slot] = arg;
      }
    }
  }
}

template <int WT, bool SPLIT, int LN, int NW, int KSLICE, int KSPLIT, int MB>
int launch_one(const LinArgs& a, bool pdl, cudaStream_t stream, bool deal = false) {
  using S = LinSmem<WT, SPLIT, LN, NW, KSLICE, KSPLIT, MB>;
  static_assert(S::TOTAL <= 227 * 1024, "tile does not fit in shared memory");
  auto kern = linear_kernel<WT, SPLIT, LN, NW, KSLICE, KSPLIT, MB>;
  // idempotent; set on every call so that it holds on every device of the process
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "linear: smem attribute: %s", cudaGetErrorString(e));
  const dim3 grid(KSPLIT, a.N / (NW * 16), deal ? (a.rows + MB - 1) / MB : 1);  // deal: MB rows per CTA
  e = launch_kernel(kern, grid, dim3(NW * 32), S::TOTAL, stream, KSPLIT, pdl, a);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "linear launch: %s", cudaGetErrorString(e));
  return 0;
}

template <int WT, bool SPLIT, int LN, int NW, int KSLICE, int KSPLIT>
int launch_mb(const LinArgs& a, bool pdl, cudaStream_t s) {
  if (a.rows <= 16) return launch_one<WT, SPLIT, LN, NW, KSLICE, KSPLIT, 16>(a, pdl, s);
  // The 64-channel tiles with K split eight ways (fc2; o, cross-o; cross-q): above 32 rows the rows are dealt over
  // several CTAs per tile that share an SM (grid.z), so that eight or more warps instead of four feed the SM's tensor
  // pipes, each CTA stages a fraction of the operand and several latency chains overlap. Measured at 64 rows: p50 step
  // 0.504 -> 0.467 ms. fc2 (K slices of 512, 140 registers): two CTAs of 32 rows; the K = 1024 ones (slices of 128, 94
  // registers): four CTAs of 16 rows, above 64 rows four of 32. (The 8-warp LayerNorm readers measured no gain from
  // dealing and keep one CTA per tile.)
  if constexpr (!SPLIT && (LN == 0 || LN == 2) && WT != B200DEC_W_BF16 && (KSLICE == 512 || KSLICE == 128) &&
                KSPLIT == 8 && NW == 4) {
    if (!a.head) {
      if (a.rows > 32 && a.rows <= 64) {
        if (KSLICE == 128) return launch_one<WT, SPLIT, LN, NW, KSLICE, KSPLIT, 16>(a, pdl, s, true);
        return launch_one<WT, SPLIT, LN, NW, KSLICE, KSPLIT, 32>(a, pdl, s, true);
      }
      // above 64 rows: four CTAs of 32 rows per tile, also for fc2 (the weights come from HBM once; a 128-row tile
      // of K slices of 512 would fill an SM's shared memory, and two passes of 64 rows would read the weights twice)
      if (a.rows > 64) return launch_one<WT, SPLIT, LN, NW, KSLICE, KSPLIT, 32>(a, pdl, s, true);
    }
  }
  if (a.rows <= 64) {
    if constexpr (LinSmem<WT, SPLIT, LN, NW, KSLICE, KSPLIT, 64>::TOTAL <= 227 * 1024)
      return launch_one<WT, SPLIT, LN, NW, KSLICE, KSPLIT, 64>(a, pdl, s);
    else
      return fail(B200DEC_EINVAL, "linear: %d rows need a smaller K / ksplit than %d for this operand", a.rows, KSLICE);
  }
  if constexpr (LinSmem<WT, SPLIT, LN, NW, KSLICE, KSPLIT, 128>::TOTAL <= 227 * 1024)
    return launch_one<WT, SPLIT, LN, NW, KSLICE, KSPLIT, 128>(a, pdl, s);
  else
    return fail(B200DEC_EINVAL, "linear: %d rows need a smaller K / ksplit than %d for this operand", a.rows, KSLICE);
}

// Does the (kind, operand, tile) combination fit shared memory for this many rows? (host-side query)
template <int WT, bool SPLIT, int LN, int NW, int KSLICE, int KSPLIT>
bool fits(int rows) {
  if (rows <= 16) return true;
  if (rows <= 64) return LinSmem<WT, SPLIT, LN, NW, KSLICE, KSPLIT, 64>::TOTAL <= 227 * 1024;
  return LinSmem<WT, SPLIT, LN, NW, KSLICE, KSPLIT, 128>::TOTAL <= 227 * 1024;
}

// the (K / ksplit, ksplit) pairs with kernels: K = 1024 as 8 x 128, 4 x 256, 2 x 512; K = 4096 as 8 x 512
#define B200_TILE_CASES(X) X(4, 128, 8) X(4, 256, 4) X(4, 512, 2) X(4, 512, 8) X(8, 128, 8) X(8, 256, 4) X(8, 512, 2) X(8, 512, 8)

template <int WT, bool SPLIT, int LN>
int launch_shape(const LinArgs& a, int warps, int k, int ksplit, bool pdl, cudaStream_t s) {
  const int kslice = k / ksplit;
  constexpr int KPB = WTraits<WT>::KPB;
#define B200_CASE(NW_, KS_, SP_)                                                                    \
  if (warps == NW_ && kslice == KS_ && ksplit == SP_) {                                             \
    if constexpr (KS_ % KPB == 0 && (!LN || KS_ * SP_ == D_MODEL) && (NW_ * 16) % (8 * SP_) == 0 && \
                  (LN != 2 || (!SPLIT && KS_ <= 256)))                                              \
      return launch_mb<WT, SPLIT, LN, NW_, KS_, SP_>(a, pdl, s);                                    \
  }
  B200_TILE_CASES(B200_CASE)
#undef B200_CASE
  return fail(B200DEC_EINVAL, "linear: no kernel for warps=%d K=%d ksplit=%d (K = 1024: 8|4|2; K = 4096: 8)", warps, k,
              ksplit);
}

template <int WT, bool SPLIT, int LN>
bool fits_shape(int warps, int k, int ksplit, int rows) {
  const int kslice = k / ksplit;
  constexpr int KPB = WTraits<WT>::KPB;
#define B200_CASE(NW_, KS_, SP_)                                                                    \
  if (warps == NW_ && kslice == KS_ && ksplit == SP_) {                                             \
    if constexpr (KS_ % KPB == 0 && (!LN || KS_ * SP_ == D_MODEL) && (NW_ * 16) % (8 * SP_) == 0 && \
                  (LN != 2 || (!SPLIT && KS_ <= 256)))                                              \
      return fits<WT, SPLIT, LN, NW_, KS_, SP_>(rows);                                              \
  }
  B200_TILE_CASES(B200_CASE)
#undef B200_CASE
  return false;
}

// one entry per weight kind, each defined in its own translation unit
int launch_int8(const LinArgs& a, bool split, int ln, int warps, int k, int ksplit, bool pdl, cudaStream_t s);
int launch_bf16(const LinArgs& a, bool split, int ln, int warps, int k, int ksplit, bool pdl, cudaStream_t s);
int launch_24(const LinArgs& a, bool split, int ln, int warps, int k, int ksplit, bool pdl, cudaStream_t s);
int launch_f16(const LinArgs& a, bool split, int ln, int warps, int k, int ksplit, bool pdl, cudaStream_t s);
bool fits_int8(bool split, int ln, int warps, int k, int ksplit, int rows);
bool fits_bf16(bool split, int ln, int warps, int k, int ksplit, int rows);
bool fits_24(bool split, int ln, int warps, int k, int ksplit, int rows);
bool fits_f16(bool split, int ln, int warps, int k, int ksplit, int rows);

}  // namespace b200dec_detail
