// Attention of one new token per row over its slot's bf16 KV cache: the step's dominant HBM stream.
//
// One CTA of 128 threads per (head, row, key split). A key (or value) vector of D = 64 / 128 bf16 is read by
// D / 8 lanes with one 16-byte load each, so a warp instruction fetches 4 (D = 64) or 2 (D = 128) whole vectors as
// contiguous 128 / 256-byte runs; each lane group walks its keys four at a time (4 key + 4 value loads in flight
// per thread, ~16 KB per CTA), with an online softmax per group in fp32 (exp2 on pre-scaled scores). The groups are
// merged in shared memory. With more than one split the partial (max, sum, output) goes to a workspace and the last
// CTA of the (row, head) to arrive merges them (a counter it then resets, so the kernel replays inside CUDA graphs;
// nobody spins). Self-attention also appends: the row's new key and value (fp32 columns of the fused qkv
// projection) are rounded to bf16 into the cache at position n[slot] and attended from registers.
//
// Cache layout (slots + 1, H, cap, D): all keys of one (slot, head) are one contiguous run, the unit a CTA streams.
#include <cooperative_groups.h>

#include "common.cuh"

using namespace b200dec_detail;
namespace cg = cooperative_groups;

namespace {

constexpr int MAX_SPLITS = 16;
constexpr int NTHREADS = 128;

DEVI float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct AttnArgs {
  const int* active;
  const float* q;  // (rows, ldq)
  __nv_bfloat16* k;
  __nv_bfloat16* v;
  const int* n;
  float* ks;         // int8 caches: one fp32 scale per cached key vector / value vector, (slots + 1, H, cap)
  float* vs;
  const int* sched;  // paired kernel: (rows, 4) = {row, slot, length, 0} by decreasing length, or null
  void* out;
  float* part;
  int* count;
  int* status;
  int ldq, H, cap, slots, out_kind, rows, splits;
  float scale_log2;  // head_dim^-0.5 * log2(e)
};


// One CTA's pass over keys [start, end) of (slot s, head h) for the query of row r, plus (with_new) the row's new key:
// on return threads tid < D hold the pass's running maximum M, sum L and un-normalised output O for dim tid.
template <int D, bool SELF>
DEVI void attend_range(const AttnArgs& p, int r, int s, int h, int n, int start, int end, bool with_new,
                       float* s_m, float* s_l, float (*s_acc)[D + 4], float& M, float& L, float& O) {
  constexpr int LPK = D / 8;           // lanes per key
  constexpr int NG = NTHREADS / LPK;   // key groups per CTA
  constexpr int U = 4;                 // keys in flight per group
  const int tid = threadIdx.x, grp = tid / LPK, gl = tid % LPK;
  const size_t base = ((size_t)s * p.H + h) * p.cap * D + gl * 8;
  const __nv_bfloat16* kb = p.k + base;
  const __nv_bfloat16* vb = p.v + base;
  // whole-warp trip count: every lane runs the same number of iterations (shuffles), invalid keys are masked
  const int first = start + (tid >> 5) * (32 / LPK);  // first key of this warp's group 0
  const int jg = grp % (32 / LPK);
  uint4 kk[U], vv[U];
  auto fetch = [&](int j0) {  // this group's U keys and values of the block of NG * U keys at j0
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int jj = j0 + jg + u * NG;
      const bool ok = jj < end;
      kk[u] = ok ? ld_stream16(kb + (size_t)jj * D) : make_uint4(0, 0, 0, 0);
      vv[u] = ok ? ld_stream16(vb + (size_t)jj * D) : make_uint4(0, 0, 0, 0);
    }
  };
  // The first block's loads go out before anything waits for the query: they depend on the schedule only, and the
  // query's round trip to L2 would otherwise stand in front of the first bytes from HBM.
  if (first < end) fetch(first);

  // the query, pre-scaled so that scores are in log2 units
  float q[8];
  {
    const float* qp = p.q + (size_t)r * p.ldq + h * D + gl * 8;
    const float4 a = ld_cg_f4(qp), b = ld_cg_f4(qp + 4);
    q[0] = a.x * p.scale_log2, q[1] = a.y * p.scale_log2, q[2] = a.z * p.scale_log2, q[3] = a.w * p.scale_log2;
    q[4] = b.x * p.scale_log2, q[5] = b.y * p.scale_log2, q[6] = b.z * p.scale_log2, q[7] = b.w * p.scale_log2;
  }
  float m = -1e30f, l = 0.f, acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;

  auto attend = [&](const uint4& kk, const uint4& vv, bool valid) {
    float d = q[0] * bf16_lo(kk.x) + q[1] * bf16_hi(kk.x) + q[2] * bf16_lo(kk.y) + q[3] * bf16_hi(kk.y) +
              q[4] * bf16_lo(kk.z) + q[5] * bf16_hi(kk.z) + q[6] * bf16_lo(kk.w) + q[7] * bf16_hi(kk.w);
#pragma unroll
    for (int o = 1; o < LPK; o <<= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
    const float sc = valid ? d : -INFINITY;
    const float mn = fmaxf(m, sc), a = ex2(m - mn), e = ex2(sc - mn);
    l = l * a + e;
    acc[0] = acc[0] * a + e * bf16_lo(vv.x), acc[1] = acc[1] * a + e * bf16_hi(vv.x);
    acc[2] = acc[2] * a + e * bf16_lo(vv.y), acc[3] = acc[3] * a + e * bf16_hi(vv.y);
    acc[4] = acc[4] * a + e * bf16_lo(vv.z), acc[5] = acc[5] * a + e * bf16_hi(vv.z);
    acc[6] = acc[6] * a + e * bf16_lo(vv.w), acc[7] = acc[7] * a + e * bf16_hi(vv.w);
    m = mn;
  };

  if (SELF && with_new && tid < 32) {
    // The new key and value: rounded to bf16 into the cache at position n, and attended as stored. `attend` shuffles
    // across the warp, so all of warp 0 goes through it with only group 0 (lanes 0 .. LPK-1) valid.
    const float* kp = p.q + (size_t)r * p.ldq + (p.H + h) * D + gl * 8;
    const float* vp = kp + p.H * D;
    const float4 k0 = ld_cg_f4(kp), k1 = ld_cg_f4(kp + 4), v0 = ld_cg_f4(vp), v1 = ld_cg_f4(vp + 4);
    const uint4 kk = make_uint4(pack_bf16(k0.x, k0.y), pack_bf16(k0.z, k0.w), pack_bf16(k1.x, k1.y),
                                pack_bf16(k1.z, k1.w));
    const uint4 vv = make_uint4(pack_bf16(v0.x, v0.y), pack_bf16(v0.z, v0.w), pack_bf16(v1.x, v1.y),
                                pack_bf16(v1.z, v1.w));
    if (grp == 0) {
      *reinterpret_cast<uint4*>(p.k + base + (size_t)n * D) = kk;
      *reinterpret_cast<uint4*>(p.v + base + (size_t)n * D) = vv;
    }
    attend(kk, vv, grp == 0);
  }

  // cached keys [start, end), group g taking start + g, + NG, ...
  for (int j0 = first; j0 < end; j0 += NG * U) {
    if (j0 != first) fetch(j0);
    const int j = j0 + jg;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (j0 + u * NG < end) attend(kk[u], vv[u], j + u * NG < end);  // warp-uniform condition
    }
  }
  // merge the groups
  __syncthreads();  // the arrays may still be read by a previous pass
  if (gl == 0) s_m[grp] = m, s_l[grp] = l;
#pragma unroll
  for (int i = 0; i < 8; ++i) s_acc[grp][gl * 8 + i] = acc[i];
  __syncthreads();
  M = -1e30f, L = 0.f, O = 0.f;
  if (tid < D) {
#pragma unroll
    for (int gi = 0; gi < NG; ++gi) M = fmaxf(M, s_m[gi]);
#pragma unroll
    for (int gi = 0; gi < NG; ++gi) {
      const float w = ex2(s_m[gi] - M);
      L += w * s_l[gi];
      O += w * s_acc[gi][tid];
    }
  }
}

// ---- int8 caches: one fp32 scale per head vector (the format of the reference's int8 mode) ---------------------------
// vector -> scale = absmax / 127 (1 when the vector is zero), q = rint(clamp(x * (1 / scale), +-127)); x ~ q * scale.
//
// Half the bytes per key only pay if the instructions per byte do not double, so this pass does its arithmetic on
// pairs: a key (or value) of D int8 is read by D / 16 lanes with one 16-byte load each; four bytes become two half2
// with two byte permutes and two subtractions (the byte, biased by 128, is the low mantissa of the half 1024 + u;
// exact); the dot product runs as half2 multiply-adds, eight products per accumulator lane, then fp32 (query
// pre-scaled and rounded to fp16); the weighted values accumulate in half2 as well (a lane group sees only
// n / 32 keys, about ten, so the sums stay short) and are merged across groups in fp32. A warp takes 4 x (32 / lanes
// per key) consecutive keys per iteration and fetches their scales with one coalesced load, handed round by shuffles.
// Against the fp64 result on the dequantised caches this costs about 1e-3 relative (fp16 products), below what the
// int8 rounding of the caches itself does; whole-step parity is tested with int8 caches on the golden sequences.
constexpr int Q8_LANE_DIMS = 16;

// 4 two's-complement bytes -> half2(q0, q1), half2(q2, q3), exact
DEVI void widen_s8x4(uint32_t w, __half2& lo, __half2& hi) {
  const uint32_t x = w ^ 0x80808080u;
  const uint32_t a = __byte_perm(x, 0x64646464u, 0x4140), b = __byte_perm(x, 0x64646464u, 0x4342);
  const __half2 off = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));  // 1024 + 128
  lo = __hsub2(*reinterpret_cast<const __half2*>(&a), off);
  hi = __hsub2(*reinterpret_cast<const __half2*>(&b), off);
}

// The same pass as attend_range over int8 caches. The row's new key and value are rounded to bf16, quantised into the
// cache, and attended in that step as the bf16 values (the quantised copy serves the later steps), as the reference
// does.
template <int D, bool SELF>
DEVI void attend_range_q8(const AttnArgs& p, int r, int s, int h, int n, int start, int end, bool with_new,
                          float* s_m, float* s_l, float (*s_acc)[D + 4], float& M, float& L, float& O) {
  constexpr int LPK = D / Q8_LANE_DIMS;  // lanes per key
  constexpr int GPW = 32 / LPK;          // keys per warp-wide load = lane groups per warp
  constexpr int U = 4;                   // keys in flight per group
  constexpr int KPW = U * GPW;           // keys per warp and iteration
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane / LPK, gl = lane % LPK;
  const int8_t* k8 = reinterpret_cast<const int8_t*>(p.k);
  const int8_t* v8 = reinterpret_cast<const int8_t*>(p.v);
  const size_t vec0 = ((size_t)s * p.H + h) * p.cap;  // index of key 0: scales, and * D the vectors

  // the lane's 16 dims of the query, pre-scaled into log2 units, as fp16 pairs
  __half2 qh[8];
  {
    const float* qp = p.q + (size_t)r * p.ldq + h * D + gl * Q8_LANE_DIMS;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 a = ld_cg_f4(qp + 4 * i);
      qh[2 * i] = __floats2half2_rn(a.x * p.scale_log2, a.y * p.scale_log2);
      qh[2 * i + 1] = __floats2half2_rn(a.z * p.scale_log2, a.w * p.scale_log2);
    }
  }
  float m = -1e30f, l = 0.f;
  __half2 acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = __float2half2_rn(0.f);

  if (SELF && with_new && tid < 32) {
    // warp 0: group 0 (lanes 0 .. LPK-1) holds the new key and value in fp32; all lanes go through the shuffles
    const float* qp = p.q + (size_t)r * p.ldq + h * D + gl * Q8_LANE_DIMS;
    const float* kp = qp + p.H * D;
    const float* vp = kp + p.H * D;
    float kn[16], vn[16], d = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 qa = ld_cg_f4(qp + 4 * i), a = ld_cg_f4(kp + 4 * i), b = ld_cg_f4(vp + 4 * i);
      const uint32_t k01 = pack_bf16(a.x, a.y), k23 = pack_bf16(a.z, a.w), v01 = pack_bf16(b.x, b.y), v23 = pack_bf16(b.z, b.w);
      kn[4 * i] = bf16_lo(k01), kn[4 * i + 1] = bf16_hi(k01), kn[4 * i + 2] = bf16_lo(k23), kn[4 * i + 3] = bf16_hi(k23);
      vn[4 * i] = bf16_lo(v01), vn[4 * i + 1] = bf16_hi(v01), vn[4 * i + 2] = bf16_lo(v23), vn[4 * i + 3] = bf16_hi(v23);
      d += (qa.x * kn[4 * i] + qa.y * kn[4 * i + 1]) + (qa.z * kn[4 * i + 2] + qa.w * kn[4 * i + 3]);
    }
    auto quantise = [&](const float (&f)[16], int8_t* dst, float* scale) {
      float mx = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) mx = fmaxf(mx, fabsf(f[i]));
#pragma unroll
      for (int o = 1; o < LPK; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float sc = mx > 0.f ? __fdiv_rn(mx, 127.f) : 1.f, inv = __fdiv_rn(1.f, sc);
      uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int qi = __float2int_rn(fminf(fmaxf(__fmul_rn(f[i], inv), -127.f), 127.f));
        w[i >> 2] |= (uint32_t)(qi & 0xff) << ((i & 3) * 8);
      }
      if (g == 0) {
        *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
        if (gl == 0) *scale = sc;
      }
    };
    quantise(kn, const_cast<int8_t*>(k8) + (vec0 + n) * D + gl * Q8_LANE_DIMS, p.ks + vec0 + n);
    quantise(vn, const_cast<int8_t*>(v8) + (vec0 + n) * D + gl * Q8_LANE_DIMS, p.vs + vec0 + n);
    d *= p.scale_log2;
#pragma unroll
    for (int o = 1; o < LPK; o <<= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
    m = d;         // every group of the warp computed the same score: the warp's running maximum starts there
    if (g == 0) {  // and one group counts the key: weight 1
      l = 1.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = __floats2half2_rn(vn[2 * i], vn[2 * i + 1]);
    }
  }

  const int8_t* kb = k8 + vec0 * D + gl * Q8_LANE_DIMS;
  const int8_t* vb = v8 + vec0 * D + gl * Q8_LANE_DIMS;
  // whole-warp trip count: every lane runs the same number of iterations (shuffles), invalid keys are masked
  for (int k0 = start + warp * KPW; k0 < end; k0 += (NTHREADS / 32) * KPW) {
    // the scales of the warp's KPW keys: lane i fetches those of key k0 + i
    float ks_l = 1.f, vs_l = 1.f;
    if (lane < KPW && k0 + lane < end) {
      ks_l = __uint_as_float(ld_stream4(p.ks + vec0 + k0 + lane));
      vs_l = __uint_as_float(ld_stream4(p.vs + vec0 + k0 + lane));
    }
    uint4 kw[U], vw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = k0 + u * GPW + g;
      const bool ok = j < end;
      kw[u] = ok ? ld_stream16(kb + (size_t)j * D) : make_uint4(0, 0, 0, 0);
      vw[u] = ok ? ld_stream16(vb + (size_t)j * D) : make_uint4(0, 0, 0, 0);
    }
    float sc[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t w[4] = {kw[u].x, kw[u].y, kw[u].z, kw[u].w};
      __half2 a0 = __float2half2_rn(0.f), a1 = a0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        __half2 lo, hi;
        widen_s8x4(w[i], lo, hi);
        a0 = __hfma2(qh[2 * i], lo, a0);
        a1 = __hfma2(qh[2 * i + 1], hi, a1);
      }
      const float2 f = __half22float2(__hadd2(a0, a1));
      float d = f.x + f.y;
#pragma unroll
      for (int o = 1; o < LPK; o <<= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      const float ksc = __shfl_sync(0xffffffffu, ks_l, u * GPW + g);
      sc[u] = (k0 + u * GPW + g < end) ? d * ksc : -INFINITY;
    }
    // one running maximum per warp (not per group): the groups' sums can be added up at the end without rescaling
    float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
#pragma unroll
    for (int o = LPK; o < 32; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    const float mn = fmaxf(m, mx);
    const float a = ex2(m - mn);
    const __half2 ah = __float2half2_rn(a);
    l *= a;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = __hmul2(acc[i], ah);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const float e = ex2(sc[u] - mn);
      const float vsc = __shfl_sync(0xffffffffu, vs_l, u * GPW + g);
      l += e;
      const __half2 eh = __float2half2_rn(e * vsc);
      const uint32_t w[4] = {vw[u].x, vw[u].y, vw[u].z, vw[u].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        __half2 lo, hi;
        widen_s8x4(w[i], lo, hi);
        acc[2 * i] = __hfma2(eh, lo, acc[2 * i]);
        acc[2 * i + 1] = __hfma2(eh, hi, acc[2 * i + 1]);
      }
    }
    m = mn;
  }
  // merge: a warp's groups share their maximum, so their sums add up (shuffles, in the accumulators' fp16 pairs); then
  // one (max, sum, output) set per warp through shared memory
#pragma unroll
  for (int o = LPK; o < 32; o <<= 1) {
    l += __shfl_xor_sync(0xffffffffu, l, o);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t other = __shfl_xor_sync(0xffffffffu, *reinterpret_cast<const uint32_t*>(&acc[i]), o);
      acc[i] = __hadd2(acc[i], *reinterpret_cast<const __half2*>(&other));
    }
  }
  __syncthreads();  // the arrays may still be read by a previous pass
  if (g == 0) {
    if (gl == 0) s_m[warp] = m, s_l[warp] = l;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float2 f = __half22float2(acc[i]);
      s_acc[warp][gl * Q8_LANE_DIMS + 2 * i] = f.x, s_acc[warp][gl * Q8_LANE_DIMS + 2 * i + 1] = f.y;
    }
  }
  __syncthreads();
  constexpr int NG = NTHREADS / 32;
  M = -1e30f, L = 0.f, O = 0.f;
  if (tid < D) {
#pragma unroll 8
    for (int gi = 0; gi < NG; ++gi) M = fmaxf(M, s_m[gi]);
#pragma unroll 8
    for (int gi = 0; gi < NG; ++gi) {
      const float w = ex2(s_m[gi] - M);
      L += w * s_l[gi];
      O += w * s_acc[gi][tid];
    }
  }
}

template <int D, bool SELF, bool Q8>
DEVI void attend_pass(const AttnArgs& p, int r, int s, int h, int n, int start, int end, bool with_new, float* s_m,
                      float* s_l, float (*s_acc)[D + 4], float& M, float& L, float& O) {
  if constexpr (Q8) attend_range_q8<D, SELF>(p, r, s, h, n, start, end, with_new, s_m, s_l, s_acc, M, L, O);
  else attend_range<D, SELF>(p, r, s, h, n, start, end, with_new, s_m, s_l, s_acc, M, L, O);
}

template <int D>
DEVI void store_out(const AttnArgs& p, int r, int h, float val) {
  const size_t o = (size_t)r * p.H * D + h * D + threadIdx.x;
  if (p.out_kind == B200DEC_OUT_F16)
    reinterpret_cast<__half*>(p.out)[o] = __float2half_rn(clamp_h(val));
  else
    reinterpret_cast<float*>(p.out)[o] = val;
}

// slot and length of row r, clamped into range (a bad value is reported through the status word)
template <bool SELF>
DEVI void row_state(const AttnArgs& p, int r, bool report, int& s, int& n) {
  s = p.active[r];
  if (s < 0 || s > p.slots) {
    if (report) atomicOr(p.status, B200DEC_ST_SLOT_RANGE);
    s = p.slots;
  }
  n = p.n[s];
  if (SELF ? (n < 0 || n >= p.cap) : (n < 1 || n > p.cap)) {
    if (report) atomicOr(p.status, SELF ? B200DEC_ST_POS_RANGE : B200DEC_ST_FRAMES_RANGE);
    n = SELF ? max(0, min(n, p.cap - 1)) : max(1, min(n, p.cap));
  }
}

template <int D, bool SELF, bool Q8>
__global__ void __launch_bounds__(NTHREADS, 7) attention_kernel(const AttnArgs p) {
  constexpr int NG = NTHREADS / (Q8 ? D / Q8_LANE_DIMS : D / 8);  // lane groups = partial (max, sum, output) sets
  __shared__ float s_m[NG], s_l[NG];
  __shared__ float s_acc[NG][D + 4];
  __shared__ int s_last;

  const int h = blockIdx.x, r = blockIdx.y, sp = blockIdx.z, nsp = p.splits;
  const int tid = threadIdx.x;
  pdl_wait();

  int s, n;
  row_state<SELF>(p, r, tid == 0, s, n);
  const int chunk = (n + nsp - 1) / nsp, start = sp * chunk, end = min(n, start + chunk);
  float M, L, O;
  attend_pass<D, SELF, Q8>(p, r, s, h, n, start, end, sp == 0, s_m, s_l, s_acc, M, L, O);
  // Dependents are released late, when this CTA's keys are done: a grid that started earlier would sit on registers
  // and shared memory the attention CTAs need for the whole stream, and it could still only begin its own work after
  // this grid's last CTA. (A kernel reads before its own wait only what was written at least two kernels earlier.)
  pdl_trigger();
  if (nsp == 1) {
    if (tid < D) store_out<D>(p, r, h, O / L);
    return;
  }
  // split: partial to the workspace, the last CTA of this (row, head) merges
  const int item = r * p.H + h;
  float* part = p.part + ((size_t)item * MAX_SPLITS + sp) * (D + 2);
  if (tid < D) part[tid] = O;
  if (tid == 0) part[D] = M, part[D + 1] = L;
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(p.count + item, 1) == nsp - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (tid < D) {
    const float* pb = p.part + (size_t)item * MAX_SPLITS * (D + 2);
    float MM = -1e30f;
    for (int i = 0; i < nsp; ++i) MM = fmaxf(MM, __ldcg(pb + i * (D + 2) + D));
    float LL = 0.f, OO = 0.f;
    for (int i = 0; i < nsp; ++i) {
      const float w = ex2(__ldcg(pb + i * (D + 2) + D) - MM);
      LL += w * __ldcg(pb + i * (D + 2) + D + 1);
      OO += w * __ldcg(pb + i * (D + 2) + tid);
    }
    store_out<D>(p, r, h, OO / LL);
  }
  if (tid == 0) p.count[item] = 0;
}

// ---- large batches: rows paired long with short --------------------------------------------------------------------
//
// With a thousand (row, head) items every SM holds several CTAs and the stream runs at memory speed while all of them
// are busy, but a row's CTA can only keep so many bytes in flight, so the longest rows decide when the kernel ends.
// Here the rows are ranked by length inside the kernel and the i-th longest is paired with the i-th shortest in a
// cluster of two CTAs: CTA 0 takes the head of the long row, CTA 1 the short row and then the tail of the long one, cut
// so that both read the same number of keys. CTA 1 hands its partial (max, sum, output) of the long row to CTA 0
// through distributed shared memory; one cluster barrier, no global workspace. Rows of (nearly) equal length skip the
// exchange.
constexpr int PAIR_MAX_ROWS = 256;

template <int D, bool SELF, bool TABLE, bool Q8>
__global__ void __launch_bounds__(NTHREADS, 7) attention_pair_kernel(const AttnArgs p) {
  constexpr int NG = NTHREADS / (Q8 ? D / Q8_LANE_DIMS : D / 8);
  __shared__ float s_m[NG], s_l[NG];
  __shared__ float s_acc[NG][D + 4];
  __shared__ float s_peer[D + 2];  // CTA 0: the partial its peer computed for the long row
  __shared__ int t_slot[TABLE ? 1 : PAIR_MAX_ROWS], t_n[TABLE ? 1 : PAIR_MAX_ROWS];
  __shared__ int s_pair[2];

  cluster_arrive_entry();  // the peer may be written to only once it has started: see cluster_wait_entry() below
  cg::cluster_group cluster = cg::this_cluster();
  const int role = blockIdx.x, h = blockIdx.y, i = blockIdx.z, rows = p.rows;
  const int tid = threadIdx.x;
  int r_long, r_short, s_long, s_short, n_long, n_short;
  if constexpr (TABLE) {
    // the step's schedule (built beside the embedding, at least two kernels ago: readable before the wait): two
    // entries, no dependent loads
    const int4 a = __ldcg(reinterpret_cast<const int4*>(p.sched) + i);
    const int4 b = __ldcg(reinterpret_cast<const int4*>(p.sched) + (rows - 1 - i));
    r_long = a.x, s_long = a.y, n_long = a.z, r_short = b.x, s_short = b.y, n_short = b.z;
    pdl_wait();
  } else {
    pdl_wait();
    for (int r = tid; r < rows; r += NTHREADS) {
      int s, n;
      row_state<SELF>(p, r, blockIdx.x + blockIdx.y + blockIdx.z == 0, s, n);
      t_slot[r] = s, t_n[r] = n;
    }
    __syncthreads();
    for (int r = tid; r < rows; r += NTHREADS) {  // rank by decreasing length, ties by row
      const int n = t_n[r];
      int rank = 0;
      for (int j = 0; j < rows; ++j) rank += (t_n[j] > n) || (t_n[j] == n && j < r);
      if (rank == i) s_pair[0] = r;
      if (rank == rows - 1 - i) s_pair[1] = r;
    }
    __syncthreads();
    r_long = s_pair[0], r_short = s_pair[1];
    s_long = t_slot[r_long], s_short = t_slot[r_short], n_long = t_n[r_long], n_short = t_n[r_short];
  }
  const bool solo = r_long == r_short;  // the middle row of an odd count
  // keys [cut, n_long) of the long row go to CTA 1 (a multiple of 16 keeps both CTAs' loads aligned to whole groups)
  int cut = n_long;
  if (!solo && n_long - n_short >= 32) cut = min(n_long, ((n_long + n_short) / 2 + 15) & ~15);
  const bool helped = cut < n_long;

  float M, L, O;
  if (role == 0) {
    attend_pass<D, SELF, Q8>(p, r_long, s_long, h, n_long, 0, cut, true, s_m, s_l, s_acc, M, L, O);
    pdl_trigger();  // late: see attention_kernel
    if (helped) {
      cluster_wait_entry();  // completes the phase opened at entry (a thread may not arrive twice in a row)
      cluster.sync();        // the peer's partial has landed
      if (tid < D) {
        const float pm = s_peer[D], pl = s_peer[D + 1], po = s_peer[tid];
        const float mm = fmaxf(M, pm), w0 = ex2(M - mm), w1 = ex2(pm - mm);
        L = w0 * L + w1 * pl, O = w0 * O + w1 * po;
      }
    }
    if (tid < D) store_out<D>(p, r_long, h, O / L);
  } else {
    if (!solo) {
      attend_pass<D, SELF, Q8>(p, r_short, s_short, h, n_short, 0, n_short, true, s_m, s_l, s_acc, M, L, O);
      if (tid < D) store_out<D>(p, r_short, h, O / L);
    }
    if (helped) {
      attend_pass<D, SELF, Q8>(p, r_long, s_long, h, n_long, cut, n_long, false, s_m, s_l, s_acc, M, L, O);
      pdl_trigger();
      cluster_wait_entry();  // CTA 0 has started (it arrived at its entry, long ago by now)
      float* peer = cluster.map_shared_rank(s_peer, 0);
      if (tid < D) peer[tid] = O;
      if (tid == 0) peer[D] = M, peer[D + 1] = L;
      cluster.sync();
    }
  }
}

int pick_splits(int rows, int heads, int cap) {
  // enough CTAs for every SM to hold several, but at least ~32 keys per split
  const int items = rows * heads;
  int s = (4 * 148 + items - 1) / items;
  const int by_len = cap / 32 > 1 ? cap / 32 : 1;
  if (s > by_len) s = by_len;
  if (s > MAX_SPLITS) s = MAX_SPLITS;
  return s < 1 ? 1 : s;
}

}  // namespace

namespace {

template <bool Q8>
cudaError_t launch_attention(bool pair, bool table, int head_dim, int self, dim3 grid, cudaStream_t s, int pdl,
                             const AttnArgs& p) {
  const dim3 block(NTHREADS);
#define B200_ATTN_CASE(D_, SELF_)                                                                                  \
  if (head_dim == D_ && (self != 0) == SELF_) {                                                                    \
    if (!pair) return launch_kernel(attention_kernel<D_, SELF_, Q8>, grid, block, 0, s, 0, pdl, p);                \
    return table ? launch_kernel(attention_pair_kernel<D_, SELF_, true, Q8>, grid, block, 0, s, 2, pdl, p)         \
                 : launch_kernel(attention_pair_kernel<D_, SELF_, false, Q8>, grid, block, 0, s, 2, pdl, p);       \
  }
  B200_ATTN_CASE(64, true)
  B200_ATTN_CASE(64, false)
  B200_ATTN_CASE(128, true)
  B200_ATTN_CASE(128, false)
#undef B200_ATTN_CASE
  return cudaErrorInvalidValue;
}

// Shared by the entry points. sched != null: the paired kernel on a row schedule; else the paired kernel with its own
// ranking for a large batch, or one CTA per (row, head, split). ks != null: int8 caches with per-vector scales.
int run_attention(const char* what, int self, const int32_t* active, const float* q, int ldq, void* kcache, void* vcache,
                  float* ks, float* vs, const int32_t* n, const int32_t* sched, int slots, int heads, int head_dim,
                  int cap, float scale, void* out, int out_kind, int rows, float* part, int32_t* count, int32_t* status,
                  int pdl, void* stream) {
  B200_REQUIRE(q && kcache && vcache && out && (sched || (active && n && status)), "%s: null pointer", what);
  B200_REQUIRE((ks == nullptr) == (vs == nullptr), "%s: key and value scales go together", what);
  B200_REQUIRE(head_dim == 64 || head_dim == 128, "%s: head_dim %d (64 or 128)", what, head_dim);
  B200_REQUIRE(rows >= 1 && rows <= 65535 && heads >= 1 && cap >= 1, "%s: rows %d heads %d cap %d", what, rows, heads,
               cap);
  B200_REQUIRE(!sched || (rows <= PAIR_MAX_ROWS && ((uintptr_t)sched & 15) == 0),
               "%s: schedule (rows <= %d, 16-byte aligned)", what, PAIR_MAX_ROWS);
  B200_REQUIRE(ldq % 4 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)kcache & 15) == 0 &&
                   ((uintptr_t)vcache & 15) == 0, "%s: alignment", what);
  B200_REQUIRE(out_kind == B200DEC_OUT_F16 || out_kind == B200DEC_OUT_F32, "%s: out_kind", what);
  AttnArgs p{};
  p.active = active, p.q = q, p.k = (__nv_bfloat16*)kcache, p.v = (__nv_bfloat16*)vcache, p.ks = ks, p.vs = vs;
  p.n = n, p.sched = sched, p.out = out, p.part = part, p.count = count, p.status = status;
  p.ldq = ldq, p.H = heads, p.cap = cap, p.slots = slots, p.out_kind = out_kind, p.rows = rows;
  p.splits = (!sched && part && count) ? pick_splits(rows, heads, cap) : 1;
  p.scale_log2 = scale * 1.4426950408889634f;
  // a large batch: rows paired long with short, two CTAs per pair and head
  const bool pair = sched || (p.splits == 1 && rows * heads >= 512 && rows <= PAIR_MAX_ROWS);
  const dim3 grid = pair ? dim3(2, heads, (rows + 1) / 2) : dim3(heads, rows, p.splits);
  const cudaStream_t st = (cudaStream_t)stream;
  const cudaError_t e = ks ? launch_attention<true>(pair, sched != nullptr, head_dim, self, grid, st, pdl, p)
                           : launch_attention<false>(pair, sched != nullptr, head_dim, self, grid, st, pdl, p);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "%s launch: %s", what, cudaGetErrorString(e));
  return 0;
}

}  // namespace

extern "C" {

int64_t b200dec_attention_scratch_floats(int rows, int heads, int head_dim) {
  return (int64_t)rows * heads * MAX_SPLITS * (head_dim + 2);
}

int b200dec_attention(int self, const int32_t* active, const float* q, int ldq, void* kcache, void* vcache,
                      const int32_t* n, int slots, int heads, int head_dim, int cap, float scale, void* out,
                      int out_kind, int rows, float* part, int32_t* count, int32_t* status, int pdl, void* stream) {
  return run_attention("attention", self, active, q, ldq, kcache, vcache, nullptr, nullptr, n, nullptr, slots, heads,
                       head_dim, cap, scale, out, out_kind, rows, part, count, status, pdl, stream);
}

int b200dec_attention_q8(int self, const int32_t* active, const float* q, int ldq, void* kcache, void* vcache,
                         float* kscale, float* vscale, const int32_t* n, int slots, int heads, int head_dim, int cap,
                         float scale, void* out, int out_kind, int rows, float* part, int32_t* count, int32_t* status,
                         int pdl, void* stream) {
  B200_REQUIRE(kscale && vscale, "attention_q8: null scales");
  return run_attention("attention_q8", self, active, q, ldq, kcache, vcache, kscale, vscale, n, nullptr, slots, heads,
                       head_dim, cap, scale, out, out_kind, rows, part, count, status, pdl, stream);
}

int b200dec_attention_paired(int self, const int32_t* sched, const float* q, int ldq, void* kcache, void* vcache,
                             int heads, int head_dim, int cap, float scale, void* out, int out_kind, int rows, int pdl,
                             void* stream) {
  B200_REQUIRE(sched, "attention_paired: null schedule");
  return run_attention("attention_paired", self, nullptr, q, ldq, kcache, vcache, nullptr, nullptr, nullptr, sched, 0,
                       heads, head_dim, cap, scale, out, out_kind, rows, nullptr, nullptr, nullptr, pdl, stream);
}

int b200dec_attention_paired_q8(int self, const int32_t* sched, const float* q, int ldq, void* kcache, void* vcache,
                                float* kscale, float* vscale, int heads, int head_dim, int cap, float scale, void* out,
                                int out_kind, int rows, int pdl, void* stream) {
  B200_REQUIRE(sched && kscale && vscale, "attention_paired_q8: null schedule or scales");
  return run_attention("attention_paired_q8", self, nullptr, q, ldq, kcache, vcache, kscale, vscale, nullptr, sched, 0,
                       heads, head_dim, cap, scale, out, out_kind, rows, nullptr, nullptr, nullptr, pdl, stream);
}

}  // extern "C"

// ---- the same attention for callers that cannot hand over scratch memory ---------------------------------------------
//
// Some hosts of this library may not allocate device memory at the point where they call it: a serving loop whose
// memory pool was sized and frozen at start-up, a plugin ABI that hands a kernel nothing but its inputs and outputs,
// a foreign-language runtime (cgo, JNI) whose bookkeeping would never see a cudaMalloc made on its behalf. For them
// the split workspace (partial outputs of a row's spans and the per-row arrival counters) lives in this file-scope
// device array instead of in a caller's buffer. Every GPU that loads the library holds its 4.3 MB until the process
// exits, which is why its capacity is kept modest: rows * heads <= 512, which covers the small batches whose rows the
// kernel splits into spans to fill the GPU (a large batch gives every CTA a whole row and needs no workspace).
namespace {
constexpr int STATIC_MAX_ITEMS = 512;                                  // rows * heads
constexpr size_t STATIC_PART_FLOATS = (size_t)STATIC_MAX_ITEMS * MAX_SPLITS * (128 + 2);  // head_dim up to 128
static __device__ __align__(256) float g_static_scratch[STATIC_PART_FLOATS + STATIC_MAX_ITEMS];
constexpr int MAX_DEVICES = 64;
}  // namespace

extern "C" int b200dec_attention_static(int self, const int32_t* active, const float* q, int ldq, void* kcache,
                                        void* vcache, const int32_t* n, int slots, int heads, int head_dim, int cap,
                                        float scale, void* out, int out_kind, int rows, int32_t* status, int pdl,
                                        void* stream) {
  B200_REQUIRE(rows >= 1 && heads >= 1 && (long long)rows * heads <= STATIC_MAX_ITEMS,
               "attention_static: rows * heads = %lld exceeds the built-in workspace of %d (use b200dec_attention with "
               "a caller-owned workspace)", (long long)rows * heads, STATIC_MAX_ITEMS);
  B200_REQUIRE(head_dim == 64 || head_dim == 128, "attention_static: head_dim %d (64 or 128)", head_dim);
  // The array's name is only a host-side handle; the device address comes from the runtime, once per device, with that
  // device current. This first call per device is the set-up and should happen before any stream capture.
  static float* base[MAX_DEVICES] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "attention_static: cudaGetDevice: %s", cudaGetErrorString(e));
  B200_REQUIRE(dev >= 0 && dev < MAX_DEVICES, "attention_static: device %d", dev);
  float* scratch = __atomic_load_n(&base[dev], __ATOMIC_ACQUIRE);
  if (!scratch) {
    e = cudaGetSymbolAddress((void**)&scratch, g_static_scratch);
    if (e != cudaSuccess || !scratch)
      return fail(B200DEC_ECUDA, "attention_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    __atomic_store_n(&base[dev], scratch, __ATOMIC_RELEASE);  // same value from every thread that races here
  }
  int32_t* count = reinterpret_cast<int32_t*>(scratch + STATIC_PART_FLOATS);
  // The array keeps whatever the previous call left. The partials are fully rewritten before they are read; the
  // arrival counters must start at zero (a call that was cut short could have left them otherwise), so clear them on
  // the caller's stream first. A memset is not an allocation.
  e = cudaMemsetAsync(count, 0, (size_t)rows * heads * sizeof(int32_t), (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "attention_static: clearing the counters: %s", cudaGetErrorString(e));
  // The kernel's predecessor on the stream is the memset above, not a kernel: there is nothing to launch it
  // programmatically after, so `pdl` is accepted for symmetry with b200dec_attention and not used.
  (void)pdl;
  return b200dec_attention(self, active, q, ldq, kcache, vcache, n, slots, heads, head_dim, cap, scale, out, out_kind,
                           rows, scratch, count, status, 0, stream);
}
