// Small-M projections of the decoding step: out (rows, N) = act(A (rows, K) x W^T * scale + bias), rows <= 128.
//
// A step's projections are bound by reading their weights once from HBM, and each one is tiny (1 - 16 MB), so the
// kernel is built around three things:
//   * Weights are the M operand of mma.sync m16n8k16 ("swap A/B": 16 output channels x the step's rows), so a warp
//     owns 16 channels and streams exactly their bytes. They are re-tiled once (tile_* kernels below) so that every
//     warp-wide 16-byte load is one contiguous 512-byte run and the bytes land in registers already in fragment
//     order: nothing goes through shared memory, and all loads of a warp's K slice are issued up front, before the
//     kernel waits for its predecessor (programmatic dependent launch), so they overlap the previous kernel's tail.
//   * K is split over the CTAs of a thread-block cluster and N over grid.y, so even a 1024 x 1024 matrix spreads over
//     128 SMs; the partial tiles are added through distributed shared memory in rank order (deterministic, no
//     workspace, no atomics), each CTA finishing 1/ksplit of the tile's channels with the fused epilogue.
//   * int8 and 2:4 weights are widened to fp16 in registers (exact), bf16 weights are used as stored; activations are
//     staged once per CTA in shared memory as fp16/bf16, either copied (a16) or split from fp32 into a high and a low
//     half (two MMAs, ~22 bits of the activation) where rounding the operand would cost greedy agreement.
//
// Tiled layouts, per block of 16 channels (tile nt) x KPB k-values (block kb), blocks ordered [nt][kb]:
//   int8   KPB = 64:  1024 B = [h: 0,1][lane: 32][16 B]; lane = 4 g + t holds channel 16 nt + g + 8 h,
//                     k = 64 kb + 16 t .. + 15, as q + 128
//   bf16   KPB = 32:  1024 B, same indexing with k = 32 kb + 8 t .. + 7 (8 bf16)
//   2:4    KPB = 128: values 1024 B = [h][lane][16 B]: byte 2 s + j (s = 0..7) = kept value j of the group of four
//                     at k = 128 kb + 4 G, G = 2 (4 (s / 2) + t) + (s & 1); selectors 256 B = [h][lane][4 B], nibble s
//                     = that group's selector (first kept position | second << 2, as kernels/sparse.py:33-37)
// In step s of a block a lane holds 4 consecutive k of its two channels: (k, k+1) is fragment slot (2t, 2t+1) and
// (k+2, k+3) slot (2t+8, 2t+9); the activation fragment of the same lane takes the same 4 k, so the permutation of K
// inside a 16-step never has to be undone.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;
using namespace b200dec_detail;

namespace {

struct LinArgs {
  const uint8_t* w;
  const uint32_t* meta;
  const float* scale;
  const float* bias;
  const void* a;
  void* out;
  float* part_max;
  int* part_idx;
  float* logits;
  int lda, ldo, rows, N, K, out_kind, act, head;
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

// WT: weight storage; SPLIT: activations fp32 split in two halves (else a16 copied); NW warps = 16 NW channels per
// CTA; KSLICE k-values per CTA; MB: rows padded to a compile-time multiple of 8.
template <int WT, bool SPLIT, int NW, int KSLICE, int MB>
__global__ void __launch_bounds__(NW * 32, 1) linear_kernel(const LinArgs p) {
  using T = WTraits<WT>;
  constexpr int KPB = T::KPB, STEPS = T::STEPS, NBLK = KSLICE / KPB, NT = NW * 32, BN = NW * 16;
  constexpr int RS = KSLICE * 2 + T::PAD;  // bytes per activation row in shared memory
  constexpr int LDR = BN + 4;              // floats per row of the partial tile
  constexpr bool BF = WT == B200DEC_W_BF16;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint32_t lut[32];
  unsigned char* a_hi = smem;
  unsigned char* a_lo = smem + MB * RS;  // SPLIT only
  float* red = reinterpret_cast<float*>(smem);

  cg::cluster_group cluster = cg::this_cluster();
  const int rank = blockIdx.x, ksplit = gridDim.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int nt16 = blockIdx.y * NW + warp;  // this warp's 16 channels
  const int k0 = rank * KSLICE;

  // ---- prologue: the warp's whole weight slice into registers (independent of the previous kernel) -------------
  uint4 wr[NBLK][2];
  uint32_t mr[WT == B200DEC_W_INT8_24 ? NBLK : 1][2];
  {
    const size_t blk0 = (size_t)nt16 * (p.K / KPB) + k0 / KPB;
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
      // byte-permute controls: dense byte p of a group takes kept byte 0/1 (even step) or 2/3 (odd step) of the
      // register when p is the first / second kept position, else the zero byte (index 4 = 0x80)
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
  pdl_trigger();
  pdl_wait();

  // ---- stage the activations of this K slice ---------------------------------------------------------------------
  const int ntiles = (p.rows + 7) >> 3;
  if constexpr (!SPLIT) {
    constexpr int CH = KSLICE / 8;  // 16-byte chunks per row
    const __half* A = reinterpret_cast<const __half*>(p.a);
    for (int i = tid; i < ntiles * 8 * CH; i += NT) {
      const int r = i / CH, c = i % CH;
      if (r < p.rows)
        cp_async16(a_hi + r * RS + c * 16, A + (size_t)r * p.lda + k0 + c * 8);
      else
        *reinterpret_cast<uint4*>(a_hi + r * RS + c * 16) = make_uint4(0, 0, 0, 0);
    }
    cp_async_wait_all();
  } else {
    constexpr int CH = KSLICE / 4;  // float4 chunks per row
    const float* A = reinterpret_cast<const float*>(p.a);
    for (int i = tid; i < ntiles * 8 * CH; i += NT) {
      const int r = i / CH, c = i % CH;
      uint2 hi = make_uint2(0, 0), lo = make_uint2(0, 0);
      if (r < p.rows) {
        const float4 v = ld_cg_f4(A + (size_t)r * p.lda + k0 + c * 4);
        if constexpr (BF) {
          const float h0 = bf16_lo(pack_bf16(v.x, 0.f)), h1 = bf16_lo(pack_bf16(v.y, 0.f));
          const float h2 = bf16_lo(pack_bf16(v.z, 0.f)), h3 = bf16_lo(pack_bf16(v.w, 0.f));
          hi = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
          lo = make_uint2(pack_bf16(v.x - h0, v.y - h1), pack_bf16(v.z - h2, v.w - h3));
        } else {
          const float c0 = clamp_h(v.x), c1 = clamp_h(v.y), c2 = clamp_h(v.z), c3 = clamp_h(v.w);
          const float h0 = __half2float(__float2half_rn(c0)), h1 = __half2float(__float2half_rn(c1));
          const float h2 = __half2float(__float2half_rn(c2)), h3 = __half2float(__float2half_rn(c3));
          hi = make_uint2(pack_f16(c0, c1), pack_f16(c2, c3));
          lo = make_uint2(pack_f16(c0 - h0, c1 - h1), pack_f16(c2 - h2, c3 - h3));
        }
      }
      *reinterpret_cast<uint2*>(a_hi + r * RS + c * 8) = hi;
      *reinterpret_cast<uint2*>(a_lo + r * RS + c * 8) = lo;
    }
  }
  __syncthreads();

  // ---- multiply -----------------------------------------------------------------------------------------------------
  float acc[MB / 8][4];
#pragma unroll
  for (int nb = 0; nb < MB / 8; ++nb)
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
    } else if constexpr (WT == B200DEC_W_BF16) {
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
    // activation fragments: row nb * 8 + g, the lane's k-values of this block
#pragma unroll
    for (int nb = 0; nb < MB / 8; ++nb) {
      if (nb < ntiles) {
        const int row = nb * 8 + g;
#pragma unroll
        for (int c = 0; c < STEPS / 2; ++c) {  // one 16-byte chunk = two steps
          int col;                             // first k of the chunk inside the slice
          if constexpr (WT == B200DEC_W_INT8) col = b * 64 + t * 16 + c * 8;
          else if constexpr (WT == B200DEC_W_BF16) col = b * 32 + t * 8;
          else col = b * 128 + (4 * c + t) * 8;
          const uint4 h = *reinterpret_cast<const uint4*>(a_hi + row * RS + col * 2);
          if constexpr (BF) {
            mma_bf16(acc[nb], af[2 * c], h.x, h.y);
            mma_bf16(acc[nb], af[2 * c + 1], h.z, h.w);
          } else {
            mma_f16(acc[nb], af[2 * c], h.x, h.y);
            mma_f16(acc[nb], af[2 * c + 1], h.z, h.w);
          }
          if constexpr (SPLIT) {
            const uint4 l = *reinterpret_cast<const uint4*>(a_lo + row * RS + col * 2);
            if constexpr (BF) {
              mma_bf16(acc[nb], af[2 * c], l.x, l.y);
              mma_bf16(acc[nb], af[2 * c + 1], l.z, l.w);
            } else {
              mma_f16(acc[nb], af[2 * c], l.x, l.y);
              mma_f16(acc[nb], af[2 * c + 1], l.z, l.w);
            }
          }
        }
      }
    }
  }
  __syncthreads();  // every warp is done with the staged activations: the partial tile takes their place

  // ---- partial tile (rows x BN) to shared memory, then the cluster adds the K slices in rank order ----------------
#pragma unroll
  for (int nb = 0; nb < MB / 8; ++nb) {
    if (nb < ntiles) {
      const int r = nb * 8 + 2 * t, c = warp * 16 + g;
      red[r * LDR + c] = acc[nb][0];
      red[(r + 1) * LDR + c] = acc[nb][1];
      red[r * LDR + c + 8] = acc[nb][2];
      red[(r + 1) * LDR + c + 8] = acc[nb][3];
    }
  }
  cluster.sync();

  const int cpr = BN / ksplit;  // channels this CTA finishes (a multiple of 8)
  const int gpr = cpr >> 2;     // float4 groups per row
  const int n0 = blockIdx.y * BN + rank * cpr;
  const int items = p.rows * gpr, padded = (items + 31) & ~31;
  for (int it = tid; it < padded; it += NT) {
    const bool live = it < items;
    const int r = live ? it / gpr : 0, c4 = live ? it % gpr : 0;
    const int ch = rank * cpr + c4 * 4;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) {
      for (int q = 0; q < ksplit; ++q) {
        const float* remote = cluster.map_shared_rank(red, q);
        const float4 v = *reinterpret_cast<const float4*>(remote + r * LDR + ch);
        s.x += v.x, s.y += v.y, s.z += v.z, s.w += v.w;
      }
      const int n = blockIdx.y * BN + ch;
      if (p.scale) {
        const float4 sc = *reinterpret_cast<const float4*>(p.scale + n);
        s.x *= sc.x, s.y *= sc.y, s.z *= sc.z, s.w *= sc.w;
      }
      if (p.bias) {
        const float4 bb = *reinterpret_cast<const float4*>(p.bias + n);
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
            const float4 x = __ldcg(o);
            s.x += x.x, s.y += x.y, s.z += x.z, s.w += x.w;
          }
          *o = s;
        }
      } else if (p.logits) {
        *reinterpret_cast<float4*>(p.logits + (size_t)r * p.N + n) = s;
      }
    }
    if (p.head) {
      // first index of the maximum over this CTA's channels of row r (NaN never wins): gpr consecutive lanes
      float best = -INFINITY;
      int arg = 0x7fffffff;
      if (live) {
        const int n = blockIdx.y * BN + ch;
        const float v[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (v[e] > best) best = v[e], arg = n + e;
      }
      for (int o = 1; o < gpr && o < 32; o <<= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ob > best || (ob == best && oa < arg)) best = ob, arg = oa;
      }
      if (live && c4 == 0) {
        const int np = (p.N / BN) * ksplit, slot = blockIdx.y * ksplit + rank;
        p.part_max[(size_t)r * np + slot] = best;
        p.part_idx[(size_t)r * np + slot] = arg;
      }
    }
  }
  (void)n0;
  cluster.sync();  // no CTA leaves while another may still read its partial tile
}

// ---- tilers (init time) ----------------------------------------------------------------------------------------------

__global__ void tile_int8_kernel(const int8_t* __restrict__ q, int n, int k, uint8_t* __restrict__ out) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)n * k) return;
  const int e = i & 15, lane = (i >> 4) & 31, h = (i >> 9) & 1;
  const size_t blk = i >> 10;
  const int kb = blk % (k / 64), nt = blk / (k / 64), g = lane >> 2, t = lane & 3;
  out[i] = (uint8_t)((int)q[(size_t)(nt * 16 + g + 8 * h) * k + kb * 64 + t * 16 + e] + 128);
}

__global__ void tile_bf16_kernel(const uint16_t* __restrict__ w, int n, int k, uint16_t* __restrict__ out) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // output element (2 bytes)
  if (i >= (size_t)n * k) return;
  const int e = i & 7, lane = (i >> 3) & 31, h = (i >> 8) & 1;
  const size_t blk = i >> 9;
  const int kb = blk % (k / 32), nt = blk / (k / 32), g = lane >> 2, t = lane & 3;
  out[i] = w[(size_t)(nt * 16 + g + 8 * h) * k + kb * 32 + t * 8 + e];
}

__global__ void tile_24_kernel(const int8_t* __restrict__ kept, const uint32_t* __restrict__ words, int n, int k,
                               uint8_t* __restrict__ out, uint32_t* __restrict__ meta) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // output value byte
  if (i >= (size_t)n * (k / 2)) return;
  const int e = i & 15, lane = (i >> 4) & 31, h = (i >> 9) & 1;
  const size_t blk = i >> 10;
  const int kb = blk % (k / 128), nt = blk / (k / 128), g = lane >> 2, t = lane & 3;
  const int row = nt * 16 + g + 8 * h;
  const int s = e >> 1, j = e & 1;
  const int G = kb * 32 + 2 * (4 * (s >> 1) + t) + (s & 1);  // group of four along K
  out[i] = (uint8_t)kept[(size_t)row * (k / 2) + 2 * G + j];
  if (e == 0) {
    uint32_t m = 0;
    for (int ss = 0; ss < 8; ++ss) {
      const int GG = kb * 32 + 2 * (4 * (ss >> 1) + t) + (ss & 1);
      const uint32_t word = words[(size_t)row * (k / 32) + (GG >> 3)];
      m |= ((word >> (4 * (GG & 7))) & 15u) << (4 * ss);
    }
    meta[blk * 64 + h * 32 + lane] = m;
  }
}

// ---- dispatch ------------------------------------------------------------------------------------------------------------

template <int WT, bool SPLIT, int NW, int KSLICE, int MB>
int launch(const LinArgs& a, int ksplit, bool pdl, cudaStream_t stream) {
  using T = WTraits<WT>;
  constexpr int RS = KSLICE * 2 + T::PAD;
  constexpr size_t a_bytes = (size_t)MB * RS * (SPLIT ? 2 : 1);
  constexpr size_t r_bytes = (size_t)MB * (NW * 16 + 4) * 4;
  constexpr size_t smem = a_bytes > r_bytes ? a_bytes : r_bytes;
  static_assert(smem <= 227 * 1024, "tile does not fit in shared memory");
  auto kern = linear_kernel<WT, SPLIT, NW, KSLICE, MB>;
  // per-instantiation, idempotent; set on every call so it holds on every device of the process
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "linear: smem attribute: %s", cudaGetErrorString(e));
  const dim3 grid(ksplit, a.N / (NW * 16));
  e = launch_kernel(kern, grid, dim3(NW * 32), smem, stream, ksplit, pdl, a);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "linear launch: %s", cudaGetErrorString(e));
  return 0;
}

template <int WT, bool SPLIT, int NW, int KSLICE>
int launch_mb(const LinArgs& a, int ksplit, bool pdl, cudaStream_t s) {
  constexpr size_t rs = KSLICE * 2 + WTraits<WT>::PAD;
  if (a.rows <= 16) return launch<WT, SPLIT, NW, KSLICE, 16>(a, ksplit, pdl, s);
  if (a.rows <= 64) return launch<WT, SPLIT, NW, KSLICE, 64>(a, ksplit, pdl, s);
  if constexpr (128 * rs * (SPLIT ? 2 : 1) <= 227 * 1024)
    return launch<WT, SPLIT, NW, KSLICE, 128>(a, ksplit, pdl, s);
  else
    return fail(B200DEC_EINVAL, "linear: %d rows of a split operand need K / ksplit <= 256", a.rows);
}

template <int WT, bool SPLIT>
int launch_shape(const LinArgs& a, int warps, int ksplit, bool pdl, cudaStream_t s) {
  const int kslice = a.K / ksplit;
  constexpr int KPB = WTraits<WT>::KPB;
#define B200_CASE(NW, KS)                                                         \
  if (warps == NW && kslice == KS) {                                              \
    if constexpr (KS % KPB == 0) return launch_mb<WT, SPLIT, NW, KS>(a, ksplit, pdl, s); \
  }
  B200_CASE(4, 128) B200_CASE(4, 256) B200_CASE(4, 512) B200_CASE(8, 128) B200_CASE(8, 256) B200_CASE(8, 512)
#undef B200_CASE
  return fail(B200DEC_EINVAL, "linear: no kernel for warps=%d K/ksplit=%d (warps 4|8, slice 128|256|512)", warps,
              kslice);
}

int run_linear(const b200dec_weight* w, const void* a, int a_kind, int lda, int rows, void* out, int out_kind,
               int ldo, int act, float* pmax, int* pidx, float* logits, int head, int pdl, void* stream) {
  B200_REQUIRE(w && w->w && a, "linear: null pointer");
  B200_REQUIRE(rows >= 1 && rows <= 128, "linear: rows %d outside 1..128", rows);
  B200_REQUIRE(w->warps == 4 || w->warps == 8, "linear: warps must be 4 or 8");
  B200_REQUIRE(w->ksplit == 1 || w->ksplit == 2 || w->ksplit == 4 || w->ksplit == 8, "linear: ksplit %d", w->ksplit);
  B200_REQUIRE(w->n % (16 * w->warps) == 0 && w->k % w->ksplit == 0, "linear: shape (%d, %d) vs tile", w->n, w->k);
  B200_REQUIRE((16 * w->warps) % (8 * w->ksplit) == 0, "linear: warps %d too few for ksplit %d", w->warps, w->ksplit);
  B200_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)w->w & 15) == 0, "linear: operands must be 16-byte aligned");
  B200_REQUIRE(lda % 8 == 0 && lda >= w->k, "linear: lda %d", lda);
  B200_REQUIRE((w->kind == B200DEC_W_BF16) == (w->scale == nullptr), "linear: scale present iff int8");
  if (!head) {
    B200_REQUIRE(out && ((uintptr_t)out & 15) == 0 && ldo % 4 == 0 && ldo >= w->n, "linear: out / ldo");
    B200_REQUIRE(out_kind >= 0 && out_kind <= 2, "linear: out_kind");
  } else {
    B200_REQUIRE(pmax && pidx, "head: null partials");
  }
  LinArgs p{};
  p.w = (const uint8_t*)w->w, p.meta = (const uint32_t*)w->meta, p.scale = w->scale, p.bias = w->bias;
  p.a = a, p.out = out, p.part_max = pmax, p.part_idx = pidx, p.logits = logits;
  p.lda = lda, p.ldo = ldo, p.rows = rows, p.N = w->n, p.K = w->k, p.out_kind = out_kind, p.act = act, p.head = head;
  cudaStream_t s = (cudaStream_t)stream;
  const bool split = a_kind == B200DEC_A_F32_SPLIT;
  B200_REQUIRE(split || a_kind == B200DEC_A_F16, "linear: a_kind %d", a_kind);
  if (split && rows > 64 && w->k / w->ksplit > 256) {
    // 128 rows of a split operand with 512 of K per CTA do not fit shared memory: two passes of up to 64 rows (the
    // weights are read twice; projections sized for this case use K / ksplit <= 256 instead)
    const int rest = rows - 64;
    const int rc = run_linear(w, a, a_kind, lda, 64, out, out_kind, ldo, act, pmax, pidx, logits, head, pdl, stream);
    if (rc) return rc;
    const size_t osz = out_kind == B200DEC_OUT_F16 ? 2 : 4;
    const int np = head ? (w->n / (16 * w->warps)) * w->ksplit : 0;
    return run_linear(w, (const char*)a + (size_t)64 * lda * 4, a_kind, lda, rest,
                      out ? (char*)out + (size_t)64 * ldo * osz : nullptr, out_kind, ldo, act,
                      pmax ? pmax + (size_t)64 * np : nullptr, pidx ? pidx + (size_t)64 * np : nullptr,
                      logits ? logits + (size_t)64 * w->n : nullptr, head, pdl, stream);
  }
  switch (w->kind) {
    case B200DEC_W_INT8:
      return split ? launch_shape<B200DEC_W_INT8, true>(p, w->warps, w->ksplit, pdl, s)
                   : launch_shape<B200DEC_W_INT8, false>(p, w->warps, w->ksplit, pdl, s);
    case B200DEC_W_INT8_24:
      B200_REQUIRE(w->meta && !split, "linear: 2:4 weights need selectors and an a16 operand");
      return launch_shape<B200DEC_W_INT8_24, false>(p, w->warps, w->ksplit, pdl, s);
    case B200DEC_W_BF16:
      B200_REQUIRE(split, "linear: bf16 weights take the split fp32 operand");
      return launch_shape<B200DEC_W_BF16, true>(p, w->warps, w->ksplit, pdl, s);
  }
  return fail(B200DEC_EINVAL, "linear: weight kind %d", w->kind);
}

}  // namespace

namespace b200dec_detail {
int linear_impl(const b200dec_weight* w, const void* a, int a_kind, int lda, int rows, void* out, int out_kind,
                int ldo, int act, int pdl, void* stream) {
  return run_linear(w, a, a_kind, lda, rows, out, out_kind, ldo, act, nullptr, nullptr, nullptr, 0, pdl, stream);
}
int head_impl(const b200dec_weight* w, const void* a, int a_kind, int lda, int rows, float* pmax, int* pidx,
              float* logits, int pdl, void* stream) {
  return run_linear(w, a, a_kind, lda, rows, nullptr, B200DEC_OUT_F32, 0, B200DEC_ACT_NONE, pmax, pidx, logits, 1, pdl,
                    stream);
}
}  // namespace b200dec_detail

extern "C" {

int b200dec_linear(const b200dec_weight* w, const void* a, int a_kind, int lda, int rows, void* out, int out_kind,
                   int ldo, int act, int pdl, void* stream) {
  return linear_impl(w, a, a_kind, lda, rows, out, out_kind, ldo, act, pdl, stream);
}

int b200dec_head_argmax(const b200dec_weight* w, const void* a, int a_kind, int lda, int rows, float* part_max,
                        int32_t* part_idx, float* logits, int pdl, void* stream) {
  return head_impl(w, a, a_kind, lda, rows, part_max, part_idx, logits, pdl, stream);
}

int b200dec_head_partials(const b200dec_weight* w) { return w ? (w->n / (16 * w->warps)) * w->ksplit : 0; }

int64_t b200dec_tiled_bytes(int kind, int n, int k) {
  if (kind == B200DEC_W_INT8) return (int64_t)n * k;
  if (kind == B200DEC_W_BF16) return (int64_t)n * k * 2;
  if (kind == B200DEC_W_INT8_24) return (int64_t)n * k / 2;
  return -1;
}
int64_t b200dec_tiled_meta_bytes(int kind, int n, int k) { return kind == B200DEC_W_INT8_24 ? (int64_t)n * k / 8 : 0; }

int b200dec_tile_int8(const int8_t* q, int n, int k, void* tiled, void* stream) {
  B200_REQUIRE(q && tiled && n % 16 == 0 && k % 64 == 0, "tile_int8: shape (%d, %d)", n, k);
  const size_t total = (size_t)n * k;
  tile_int8_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(q, n, k, (uint8_t*)tiled);
  return check_launch("tile_int8");
}
int b200dec_tile_bf16(const void* w, int n, int k, void* tiled, void* stream) {
  B200_REQUIRE(w && tiled && n % 16 == 0 && k % 32 == 0, "tile_bf16: shape (%d, %d)", n, k);
  const size_t total = (size_t)n * k;
  tile_bf16_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>((const uint16_t*)w, n, k,
                                                                                      (uint16_t*)tiled);
  return check_launch("tile_bf16");
}
int b200dec_tile_24(const int8_t* kept, const int32_t* words, int n, int k, void* tiled, void* meta, void* stream) {
  B200_REQUIRE(kept && words && tiled && meta && n % 16 == 0 && k % 128 == 0, "tile_24: shape (%d, %d)", n, k);
  const size_t total = (size_t)n * (k / 2);
  tile_24_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      kept, (const uint32_t*)words, n, k, (uint8_t*)tiled, (uint32_t*)meta);
  return check_launch("tile_24");
}

}  // extern "C"
