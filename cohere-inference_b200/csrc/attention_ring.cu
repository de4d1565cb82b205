// Attention of one new token per row over its slot's bf16 KV cache: the step's dominant HBM stream.
//
// Persistent kernel, two CTAs per SM, built so that few warps keep many bytes in flight and leave most of each SM's
// registers and shared memory to whatever runs beside it (another row range's projections):
//   * Work units are (row, head, span of up to 128 keys), dealt to the CTAs round-robin, span-major, so every CTA gets
//     the same mix of full and partial spans whatever the rows' ragged lengths are. A unit whose span lies beyond the
//     row's length is skipped by everybody.
//   * One producer lane streams each unit's keys and values in chunks of 4 KB (32 keys of 64 dims, 16 of 128) with
//     cp.async.bulk into a ring of shared-memory stages guarded by full/empty mbarriers; the ring runs ahead across
//     unit boundaries, so the stream never drains between units. A (slot, head)'s keys are one contiguous run in
//     the cache layout (slots + 1, H, cap, D), which is what makes each chunk a single bulk copy.
//   * Four consumer warps each take a quarter of a chunk's keys, D / 16 lanes per key (each lane two 16-byte pieces
//     of the vector; for D = 64 odd keys take the pieces in the other order so that the eight lanes of a
//     shared-memory wavefront hit different banks). Scores, an online softmax per warp in fp32 (exp2 on pre-scaled
//     scores; the running maximum is warp-wide, so accumulators are rescaled only when it moves) and the weighted
//     sum of values all stay in registers; the warps' partials are merged once per unit through shared memory.
//   * A row with several spans leaves (max, sum, output) partials in a workspace; the last unit of the (row, head) to
//     finish merges them in span order (a counter it then resets, so the kernel replays inside CUDA graphs).
//   * Self-attention also appends: the row's new key and value (fp32 columns of the fused qkv projection) are
//     rounded to bf16 into the cache at position n[slot] and attended from registers by the first span's unit.
// Every mbarrier wait is bounded: a wait that runs out sets B200DEC_ST_TIMEOUT in the status word and the CTA winds
// down (the producer first waits, again bounded, for the copies it has in flight).
#include <cstdlib>

#include "common.cuh"

using namespace b200dec_detail;

namespace {

constexpr int MAX_SPLITS = 16;  // spans per (row, head) the workspace holds
#ifndef B200_ATTN_NCW
#define B200_ATTN_NCW 4
#endif
#ifndef B200_ATTN_RND
#define B200_ATTN_RND 2
#endif
constexpr int NCW = B200_ATTN_NCW;  // consumer warps
constexpr int RND = B200_ATTN_RND;  // rounds per chunk: keys in flight per lane group
constexpr int NTHREADS = (NCW + 1) * 32;
constexpr int MAX_STAGE = 16;  // ring stages (run-time choice up to this many)
constexpr int CHUNK_BYTES = RND * NCW * 1024;  // keys of one chunk (and as many bytes of values): a warp's round is 1 KB
constexpr uint32_t WAIT_LIMIT = 1u << 20;  // polls of a wait before it gives up (each poll may itself block briefly)

struct AttnArgs {
  const int* active;
  const float* q;  // (rows, ldq)
  __nv_bfloat16* k;
  __nv_bfloat16* v;
  const int* n;
  void* out;
  float* part;
  int* count;
  int* status;
  int ldq, H, cap, slots, out_kind, rows, nspan, span, nstage;
  float scale_log2;  // head_dim^-0.5 * log2(e)
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
// bounded wait for the phase with the given parity to complete; false when the limit ran out
DEVI bool mbar_wait(uint64_t* bar, uint32_t parity) {
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
DEVI void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(NCW * 32) : "memory"); }


DEVI float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// the keys of a unit: row r, head h, span sp -> [k0, k1) of the cached keys. Returns false for a unit beyond the
// row's length (nothing to do). t_slot / t_n: the rows' slots and lengths, t_order: rows by decreasing length.
struct Unit {
  int r, h, sp, s, n, k0, k1, nspans, nchunks;
};
template <int CK>
DEVI bool decode_unit(const AttnArgs& p, const int* t_slot, const int* t_n, const int* t_order, int u, Unit& w) {
  const int items = p.rows * p.H;
  w.sp = u / items;
  const int item = u - w.sp * items;
  w.r = t_order[item / p.H], w.h = item % p.H;
  w.s = t_slot[w.r], w.n = t_n[w.r];
  w.k0 = w.sp * p.span, w.k1 = min(w.n, w.k0 + p.span);
  w.nspans = max(1, (w.n + p.span - 1) / p.span);
  w.nchunks = max(1, (w.k1 - w.k0 + CK - 1) / CK);  // the first chunk also carries the query, even with no keys
  return w.sp < w.nspans;
}
// Units are dealt in passes of gridDim.x, alternate passes in reverse CTA order (a snake), rows sorted by decreasing
// length: every CTA gets long and short rows, and the CTAs that get one unit more get the shortest ones.
DEVI int unit_of_pass(int pass, int total) {
  const int G = gridDim.x, c = (pass & 1) ? G - 1 - (int)blockIdx.x : (int)blockIdx.x;
  const int u = pass * G + c;
  return u < total ? u : -1;
}

template <int D, bool SELF>
__global__ void __launch_bounds__(NTHREADS, 2) attention_kernel(const AttnArgs p) {
  constexpr int LPK = D / 16;         // lanes per key: each lane holds two 16-byte pieces (8 dims each)
  constexpr int KPW = 32 / LPK;       // keys a warp handles per round
  constexpr int CK = RND * NCW * KPW; // keys per chunk
  constexpr int KEY_BYTES = D * 2;
  static_assert(CK * KEY_BYTES == CHUNK_BYTES, "chunk size");
  constexpr bool ROT = D == 64;       // odd keys read their pieces in the other order (bank conflicts)
  constexpr int AUX = (SELF ? 3 : 1) * D;  // floats beside a unit's first chunk: the query (and the new key, value)
  // dynamic shared memory: nstage stages of [keys | values | AUX floats]
  constexpr int STAGE_BYTES = 2 * CHUNK_BYTES + AUX * 4;
  extern __shared__ __align__(128) unsigned char ring_mem[];
  const int NSTAGE = p.nstage;
  auto ring_k = [&](int st) { return ring_mem + (size_t)st * STAGE_BYTES; };
  auto ring_v = [&](int st) { return ring_mem + (size_t)st * STAGE_BYTES + CHUNK_BYTES; };
  auto aux_of = [&](int st) { return reinterpret_cast<float*>(ring_mem + (size_t)st * STAGE_BYTES + 2 * CHUNK_BYTES); };
  __shared__ __align__(8) uint64_t full[MAX_STAGE], empty[MAX_STAGE];
  __shared__ float w_m[NCW], w_l[NCW], w_acc[NCW][D];
  __shared__ int t_slot[128], t_n[128], t_order[128];
  __shared__ int s_last;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int total = p.rows * p.H * p.nspan;
  const int passes = (total + gridDim.x - 1) / gridDim.x;
  if (tid == 0) {
    for (int i = 0; i < NSTAGE; ++i) mbar_init(&full[i], 1), mbar_init(&empty[i], NCW);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_wait();     // a dependent grid may start only after this one has seen its predecessor complete, so what a
  pdl_trigger();  // kernel reads before its own wait was written at least two kernels earlier
  if (tid < p.rows) {  // the rows' slots and lengths, validated once
    int s = p.active[tid];
    if (s < 0 || s > p.slots) {
      if (blockIdx.x == 0) atomicOr(p.status, B200DEC_ST_SLOT_RANGE);
      s = p.slots;
    }
    int n = p.n[s];
    if (SELF ? (n < 0 || n >= p.cap) : (n < 1 || n > p.cap)) {
      if (blockIdx.x == 0) atomicOr(p.status, SELF ? B200DEC_ST_POS_RANGE : B200DEC_ST_FRAMES_RANGE);
      n = SELF ? max(0, min(n, p.cap - 1)) : max(1, min(n, p.cap));
    }
    t_slot[tid] = s, t_n[tid] = n;
  }
  __syncthreads();
  if (tid < p.rows) {  // rank of this row by decreasing length (ties by row)
    const int n = t_n[tid];
    int rank = 0;
    for (int j = 0; j < p.rows; ++j) rank += (t_n[j] > n) || (t_n[j] == n && j < tid);
    t_order[rank] = tid;
  }
  __syncthreads();

  if (warp == NCW) {
    // ---- producer: one lane streams the chunks of this CTA's units through the ring ---------------------------------
    if (lane != 0) return;
    uint32_t it = 0;
    bool ok = true;
    for (int pass = 0; pass < passes && ok; ++pass) {
      const int u = unit_of_pass(pass, total);
      Unit w;
      if (u < 0 || !decode_unit<CK>(p, t_slot, t_n, t_order, u, w)) continue;
      const size_t base = ((size_t)w.s * p.H + w.h) * p.cap * D;
      for (int c = 0; c < w.nchunks; ++c, ++it) {
        const int st = it % NSTAGE, j = w.k0 + c * CK;
        ok = mbar_wait(&empty[st], ((it / NSTAGE) & 1) ^ 1);
        if (!ok) break;
        const uint32_t bytes = (uint32_t)max(0, min(CK, w.k1 - j)) * KEY_BYTES;
        const bool kv_new = SELF && w.sp == 0;
        const uint32_t aux_bytes = c == 0 ? (kv_new ? 3 : 1) * D * 4 : 0;
        mbar_expect_tx(&full[st], 2 * bytes + aux_bytes);
        if (bytes) {
          bulk_load(ring_k(st), p.k + base + (size_t)j * D, bytes, &full[st]);
          bulk_load(ring_v(st), p.v + base + (size_t)j * D, bytes, &full[st]);
        }
        if (c == 0) {
          const float* qp = p.q + (size_t)w.r * p.ldq + w.h * D;
          bulk_load(aux_of(st), qp, D * 4, &full[st]);
          if (kv_new) {
            bulk_load(aux_of(st) + D, qp + p.H * D, D * 4, &full[st]);
            bulk_load(aux_of(st) + 2 * D, qp + 2 * p.H * D, D * 4, &full[st]);
          }
        }
      }
    }
    if (!ok) {
      atomicOr(p.status, B200DEC_ST_TIMEOUT);
      // the copies already issued must land before this CTA's shared memory is given away
      const uint32_t issued = it < (uint32_t)NSTAGE ? it : (uint32_t)NSTAGE;
      for (uint32_t i = 0; i < issued; ++i) {
        const uint32_t jt = it - 1 - i;
        mbar_wait(&full[jt % NSTAGE], (jt / NSTAGE) & 1);
      }
    }
    return;
  }

  // ---- consumers ----------------------------------------------------------------------------------------------------------
  const int kg = lane / LPK, ql = lane % LPK;  // key within the warp's group, lane within the key
  const int pa = ROT ? ((ql + 4 * (kg & 1)) & 7) : ql, pb = ROT ? (pa ^ 4) : (ql + LPK);  // this lane's two pieces
  uint32_t it = 0;
  bool dead = false;  // set when a bounded wait ran out: the warp then only keeps the consumers' barrier pattern
  for (int pass = 0; pass < passes; ++pass) {
    const int u = unit_of_pass(pass, total);
    Unit w;
    if (u < 0 || !decode_unit<CK>(p, t_slot, t_n, t_order, u, w)) continue;
    float qa[8], qb[8];
    float m = -1e30f, l = 0.f, acca[8], accb[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acca[i] = 0.f, accb[i] = 0.f, qa[i] = 0.f, qb[i] = 0.f;

    // RND keys per lane group at once (pieces ka, kb of each key and va, vb of its value): scores over each key's
    // lanes, one warp-wide maximum for all of them, then the accumulation; `valid` masks keys past the span's end
    auto attend = [&](const uint4 (&ka)[RND], const uint4 (&kb)[RND], const uint4 (&va)[RND], const uint4 (&vb)[RND],
                      const bool (&valid)[RND]) {
      float sc[RND];
#pragma unroll
      for (int r = 0; r < RND; ++r) {
        float d0 = qa[0] * bf16_lo(ka[r].x) + qa[1] * bf16_hi(ka[r].x), d1 = qa[2] * bf16_lo(ka[r].y) + qa[3] * bf16_hi(ka[r].y);
        float d2 = qa[4] * bf16_lo(ka[r].z) + qa[5] * bf16_hi(ka[r].z), d3 = qa[6] * bf16_lo(ka[r].w) + qa[7] * bf16_hi(ka[r].w);
        d0 += qb[0] * bf16_lo(kb[r].x) + qb[1] * bf16_hi(kb[r].x), d1 += qb[2] * bf16_lo(kb[r].y) + qb[3] * bf16_hi(kb[r].y);
        d2 += qb[4] * bf16_lo(kb[r].z) + qb[5] * bf16_hi(kb[r].z), d3 += qb[6] * bf16_lo(kb[r].w) + qb[7] * bf16_hi(kb[r].w);
        sc[r] = (d0 + d1) + (d2 + d3);
      }
#pragma unroll
      for (int o = 1; o < LPK; o <<= 1)
#pragma unroll
        for (int r = 0; r < RND; ++r) sc[r] += __shfl_xor_sync(0xffffffffu, sc[r], o);
      float mx = -INFINITY;
#pragma unroll
      for (int r = 0; r < RND; ++r) {
        sc[r] = valid[r] ? sc[r] : -INFINITY;
        mx = fmaxf(mx, sc[r]);
      }
#pragma unroll
      for (int o = LPK; o < 32; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      if (mx > m) {  // warp-uniform: the running maximum moved
        const float a = ex2(m - mx);
        l *= a;
#pragma unroll
        for (int i = 0; i < 8; ++i) acca[i] *= a, accb[i] *= a;
        m = mx;
      }
#pragma unroll
      for (int r = 0; r < RND; ++r) {
        if (valid[r]) {  // per lane: a masked key's bytes may be stale shared memory (even NaN patterns)
          const float e = ex2(sc[r] - m);
          l += e;
          acca[0] += e * bf16_lo(va[r].x), acca[1] += e * bf16_hi(va[r].x), acca[2] += e * bf16_lo(va[r].y);
          acca[3] += e * bf16_hi(va[r].y), acca[4] += e * bf16_lo(va[r].z), acca[5] += e * bf16_hi(va[r].z);
          acca[6] += e * bf16_lo(va[r].w), acca[7] += e * bf16_hi(va[r].w);
          accb[0] += e * bf16_lo(vb[r].x), accb[1] += e * bf16_hi(vb[r].x), accb[2] += e * bf16_lo(vb[r].y);
          accb[3] += e * bf16_hi(vb[r].y), accb[4] += e * bf16_lo(vb[r].z), accb[5] += e * bf16_hi(vb[r].z);
          accb[6] += e * bf16_lo(vb[r].w), accb[7] += e * bf16_hi(vb[r].w);
        }
      }
    };

    for (int c = 0; c < w.nchunks; ++c, ++it) {
      if (dead) continue;  // a wait ran out earlier: keep the barrier pattern, skip the work
      const int st = it % NSTAGE, j = w.k0 + c * CK;
      const bool got = mbar_wait(&full[st], (it / NSTAGE) & 1);
      if (!got) {
        dead = true;
        atomicOr(p.status, B200DEC_ST_TIMEOUT);
        continue;
      }
      uint4 ka[RND], kb[RND], va[RND], vb[RND];
      bool valid[RND];
#pragma unroll
      for (int r = 0; r < RND; ++r) {
        const int key = r * NCW * KPW + warp * KPW + kg;  // this lane's key of round r within the chunk
        const unsigned char* kc = ring_k(st) + key * KEY_BYTES;
        const unsigned char* vc = ring_v(st) + key * KEY_BYTES;
        ka[r] = *reinterpret_cast<const uint4*>(kc + pa * 16), kb[r] = *reinterpret_cast<const uint4*>(kc + pb * 16);
        va[r] = *reinterpret_cast<const uint4*>(vc + pa * 16), vb[r] = *reinterpret_cast<const uint4*>(vc + pb * 16);
        valid[r] = j + key < w.k1;
      }
      uint4 nka[RND], nkb[RND], nva[RND], nvb[RND];  // slot 0: the appended key / value pieces
      const bool append = SELF && c == 0 && w.sp == 0 && warp == 0;
      if (c == 0) {
        // the query's dims of this lane's two pieces, pre-scaled so that scores are in log2 units
        const float* qs = aux_of(st);
        const float4 a0 = *reinterpret_cast<const float4*>(qs + pa * 8), a1 = *reinterpret_cast<const float4*>(qs + pa * 8 + 4);
        const float4 b0 = *reinterpret_cast<const float4*>(qs + pb * 8), b1 = *reinterpret_cast<const float4*>(qs + pb * 8 + 4);
        const float sc = p.scale_log2;
        qa[0] = a0.x * sc, qa[1] = a0.y * sc, qa[2] = a0.z * sc, qa[3] = a0.w * sc;
        qa[4] = a1.x * sc, qa[5] = a1.y * sc, qa[6] = a1.z * sc, qa[7] = a1.w * sc;
        qb[0] = b0.x * sc, qb[1] = b0.y * sc, qb[2] = b0.z * sc, qb[3] = b0.w * sc;
        qb[4] = b1.x * sc, qb[5] = b1.y * sc, qb[6] = b1.z * sc, qb[7] = b1.w * sc;
        if (append) {
          auto piece = [&](const float* src, int pc) {
            const float4 x0 = *reinterpret_cast<const float4*>(src + pc * 8);
            const float4 x1 = *reinterpret_cast<const float4*>(src + pc * 8 + 4);
            return make_uint4(pack_bf16(x0.x, x0.y), pack_bf16(x0.z, x0.w), pack_bf16(x1.x, x1.y), pack_bf16(x1.z, x1.w));
          };
          nka[0] = piece(qs + D, pa), nkb[0] = piece(qs + D, pb), nva[0] = piece(qs + 2 * D, pa), nvb[0] = piece(qs + 2 * D, pb);
#pragma unroll
          for (int r = 1; r < RND; ++r) nka[r] = nka[0], nkb[r] = nkb[0], nva[r] = nva[0], nvb[r] = nvb[0];
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[st]);  // the stage's bytes are in registers
      if (append) {
        // The new key and value: rounded to bf16 into the cache at position n, and attended as stored, by the lanes
        // of key 0 of warp 0 (the other lanes and rounds go through `attend` masked: its shuffles need the whole warp).
        if (kg == 0) {
          const size_t at = (((size_t)w.s * p.H + w.h) * p.cap + w.n) * D;
          *reinterpret_cast<uint4*>(p.k + at + pa * 8) = nka[0];
          *reinterpret_cast<uint4*>(p.k + at + pb * 8) = nkb[0];
          *reinterpret_cast<uint4*>(p.v + at + pa * 8) = nva[0];
          *reinterpret_cast<uint4*>(p.v + at + pb * 8) = nvb[0];
        }
        bool nvalid[RND];
#pragma unroll
        for (int r = 0; r < RND; ++r) nvalid[r] = r == 0 && kg == 0;
        attend(nka, nkb, nva, nvb, nvalid);
      }
      if (j + warp * KPW < w.k1) attend(ka, kb, va, vb, valid);  // warp-uniform: the warp's first key is live
    }

    // ---- merge: the warp's keys (lanes with the same pieces), then the four warps ----------------------------------
#pragma unroll
    for (int o = LPK; o < 32; o <<= 1) {
      l += __shfl_xor_sync(0xffffffffu, l, o);
      const bool swap = ROT && o == LPK;  // for D = 64 the neighbouring key holds the same dims in the other order
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float oa = __shfl_xor_sync(0xffffffffu, acca[i], o), ob = __shfl_xor_sync(0xffffffffu, accb[i], o);
        acca[i] += swap ? ob : oa;
        accb[i] += swap ? oa : ob;
      }
    }
    if (kg == 0) {  // these lanes now hold the warp's sums for their pieces (l: once per key, summed over the keys)
      if (ql == 0) w_m[warp] = m, w_l[warp] = l;
#pragma unroll
      for (int i = 0; i < 8; ++i) w_acc[warp][pa * 8 + i] = acca[i], w_acc[warp][pb * 8 + i] = accb[i];
    }
    consumer_sync();
    const int item = w.r * p.H + w.h;
    float M = -1e30f, L = 0.f, O = 0.f;
    if (tid < D) {
#pragma unroll
      for (int i = 0; i < NCW; ++i) M = fmaxf(M, w_m[i]);
#pragma unroll
      for (int i = 0; i < NCW; ++i) {
        const float sc = ex2(w_m[i] - M);
        L += sc * w_l[i];
        O += sc * w_acc[i][tid];
      }
    }
    auto store = [&](float val) {
      const size_t o = (size_t)w.r * p.H * D + w.h * D + tid;
      if (p.out_kind == B200DEC_OUT_F16)
        reinterpret_cast<__half*>(p.out)[o] = __float2half_rn(clamp_h(val));
      else
        reinterpret_cast<float*>(p.out)[o] = val;
    };
    if (w.nspans == 1) {
      if (tid < D) store(O / L);
    } else {
      // partial to the workspace; the last unit of this (row, head) to arrive merges the spans in order
      float* part = p.part + ((size_t)item * MAX_SPLITS + w.sp) * (D + 2);
      if (tid < D) part[tid] = O;
      if (tid == 0) part[D] = M, part[D + 1] = L;
      __threadfence();
      consumer_sync();
      if (tid == 0) s_last = atomicAdd(p.count + item, 1) == w.nspans - 1;
      consumer_sync();
      if (s_last) {
        __threadfence();
        if (tid < D) {
          const float* pb_ = p.part + (size_t)item * MAX_SPLITS * (D + 2);
          float MM = -1e30f;
          for (int i = 0; i < w.nspans; ++i) MM = fmaxf(MM, __ldcg(pb_ + i * (D + 2) + D));
          float LL = 0.f, OO = 0.f;
          for (int i = 0; i < w.nspans; ++i) {
            const float sc = ex2(__ldcg(pb_ + i * (D + 2) + D) - MM);
            LL += sc * __ldcg(pb_ + i * (D + 2) + D + 1);
            OO += sc * __ldcg(pb_ + i * (D + 2) + tid);
          }
          store(OO / LL);
        }
        if (tid == 0) p.count[item] = 0;
      }
    }
    consumer_sync();  // w_m / w_l / w_acc / s_last are free for the next unit
  }
}

}  // namespace

extern "C" {

int b200dec_attention_ring(int self, const int32_t* active, const float* q, int ldq, void* kcache, void* vcache,
                      const int32_t* n, int slots, int heads, int head_dim, int cap, float scale, void* out,
                      int out_kind, int rows, float* part, int32_t* count, int32_t* status, int pdl, void* stream) {
  B200_REQUIRE(active && q && kcache && vcache && n && out && status, "attention_ring: null pointer");
  B200_REQUIRE(head_dim == 64 || head_dim == 128, "attention_ring: head_dim %d (64 or 128)", head_dim);
  B200_REQUIRE(rows >= 1 && rows <= 128 && heads >= 1 && cap >= 1, "attention_ring: rows %d (1..128) heads %d cap %d", rows,
               heads, cap);
  B200_REQUIRE(ldq % 4 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)kcache & 15) == 0 &&
                   ((uintptr_t)vcache & 15) == 0, "attention_ring: alignment");
  B200_REQUIRE(out_kind == B200DEC_OUT_F16 || out_kind == B200DEC_OUT_F32, "attention_ring: out_kind");
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  constexpr int per_sm = 2;  // CTAs per SM, four ring stages each (the measured optimum of 1-4 CTAs x 2-8 stages)
  // Units are whole (row, head) caches when there are enough of them to fill every CTA; a small batch splits each
  // cache into spans (multiples of a chunk) whose partials the last span to finish merges.
  const int ck = CHUNK_BYTES / (head_dim * 2), items = rows * heads;
  int nspan = (per_sm * sms + items - 1) / items;
  const int max_span = (cap + ck - 1) / ck;  // no more spans than chunks
  if (nspan > max_span) nspan = max_span;
  if (nspan > MAX_SPLITS) nspan = MAX_SPLITS;
  if (nspan < 1 || !part || !count) nspan = 1;
  const int span = ((cap + nspan - 1) / nspan + ck - 1) / ck * ck;
  nspan = (cap + span - 1) / span;
  AttnArgs p{};
  p.active = active, p.q = q, p.k = (__nv_bfloat16*)kcache, p.v = (__nv_bfloat16*)vcache, p.n = n, p.out = out;
  p.part = part, p.count = count, p.status = status;
  p.ldq = ldq, p.H = heads, p.cap = cap, p.slots = slots, p.out_kind = out_kind, p.rows = rows, p.nspan = nspan;
  p.span = span;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.nstage = 4;
  const size_t smem = (size_t)p.nstage * (2 * CHUNK_BYTES + (self ? 3 : 1) * head_dim * 4);
  const long long units = (long long)rows * heads * nspan;
  const dim3 grid((unsigned)(units < (long long)per_sm * sms ? units : (long long)per_sm * sms));
  cudaStream_t s = (cudaStream_t)stream;
  auto go = [&](auto kern) -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return e != cudaSuccess ? e : launch_kernel(kern, grid, dim3(NTHREADS), smem, s, 0, pdl, p);
  };
  cudaError_t e;
  if (head_dim == 64) e = self ? go(attention_kernel<64, true>) : go(attention_kernel<64, false>);
  else e = self ? go(attention_kernel<128, true>) : go(attention_kernel<128, false>);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "attention_ring launch: %s", cudaGetErrorString(e));
  return 0;
}

}  // extern "C"
