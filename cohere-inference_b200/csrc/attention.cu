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
  const int* sched;  // paired kernel: (rows, 4) = {row, slot, length, 0} by decreasing length, or null
  void* out;
  float* part;
  int* count;
  int* status;
  int ldq, H, cap, slots, out_kind, rows, splits;
  float scale_log2;  // head_dim^-0.5 * log2(e)
#ifdef B200DEC_STAMPS
  long long* stamps;  // per CTA 12 timer values (latency studies only)
#endif
};

#ifdef B200DEC_STAMPS
#define ATTN_STAMP(i)                                                                                               \
  do {                                                                                                              \
    if (p.stamps && threadIdx.x == 0)                                                                               \
      p.stamps[((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 12 + (i)] = stamp_clock();         \
  } while (0)
#else
#define ATTN_STAMP(i)
#endif

// One CTA's pass over keys [start, end) of (slot s, head h) for the query of row r, plus (with_new) the row's new key:
// on return threads tid < D hold the pass's running maximum M, sum L and un-normalised output O for dim tid.
template <int D, bool SELF>
DEVI void attend_range(const AttnArgs& p, int r, int s, int h, int n, int start, int end, bool with_new,
                       float* s_m, float* s_l, float (*s_acc)[D + 4], float& M, float& L, float& O) {
  constexpr int LPK = D / 8;           // lanes per key
  constexpr int NG = NTHREADS / LPK;   // key groups per CTA
  constexpr int U = 4;                 // keys in flight per group
  const int tid = threadIdx.x, grp = tid / LPK, gl = tid % LPK;

  // the query, pre-scaled so that scores are in log2 units
  float q[8];
  {
    const float* qp = p.q + (size_t)r * p.ldq + h * D + gl * 8;
    const float4 a = ld_cg_f4(qp), b = ld_cg_f4(qp + 4);
    q[0] = a.x * p.scale_log2, q[1] = a.y * p.scale_log2, q[2] = a.z * p.scale_log2, q[3] = a.w * p.scale_log2;
    q[4] = b.x * p.scale_log2, q[5] = b.y * p.scale_log2, q[6] = b.z * p.scale_log2, q[7] = b.w * p.scale_log2;
  }
  const size_t base = ((size_t)s * p.H + h) * p.cap * D + gl * 8;
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
  const __nv_bfloat16* kb = p.k + base;
  const __nv_bfloat16* vb = p.v + base;
  // whole-warp trip count: every lane runs the same number of iterations (shuffles), invalid keys are masked
  const int first = start + (tid >> 5) * (32 / LPK);  // first key of this warp's group 0
  for (int j0 = first; j0 < end; j0 += NG * U) {
    const int j = j0 + (grp % (32 / LPK));
    uint4 kk[U], vv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int jj = j + u * NG;
      const bool ok = jj < end;
      kk[u] = ok ? ld_stream16(kb + (size_t)jj * D) : make_uint4(0, 0, 0, 0);
      vv[u] = ok ? ld_stream16(vb + (size_t)jj * D) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (j0 + u * NG < end) attend(kk[u], vv[u], j + u * NG < end);  // warp-uniform condition
    }
  }
  ATTN_STAMP(3);
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

template <int D, bool SELF>
__global__ void __launch_bounds__(NTHREADS, 7) attention_kernel(const AttnArgs p) {
  constexpr int NG = NTHREADS / (D / 8);
  __shared__ float s_m[NG], s_l[NG];
  __shared__ float s_acc[NG][D + 4];
  __shared__ int s_last;

  const int h = blockIdx.x, r = blockIdx.y, sp = blockIdx.z, nsp = p.splits;
  const int tid = threadIdx.x;
  ATTN_STAMP(0);
  pdl_wait();     // a dependent grid may start only after this one has seen its predecessor complete, so what a
  pdl_trigger();  // kernel reads before its own wait was written at least two kernels earlier

  int s, n;
  row_state<SELF>(p, r, tid == 0, s, n);
  ATTN_STAMP(2);
  const int chunk = (n + nsp - 1) / nsp, start = sp * chunk, end = min(n, start + chunk);
  float M, L, O;
  attend_range<D, SELF>(p, r, s, h, n, start, end, sp == 0, s_m, s_l, s_acc, M, L, O);
  if (nsp == 1) {
    if (tid < D) store_out<D>(p, r, h, O / L);
    ATTN_STAMP(7);
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

template <int D, bool SELF, bool TABLE>
__global__ void __launch_bounds__(NTHREADS, 7) attention_pair_kernel(const AttnArgs p) {
  constexpr int NG = NTHREADS / (D / 8);
  __shared__ float s_m[NG], s_l[NG];
  __shared__ float s_acc[NG][D + 4];
  __shared__ float s_peer[D + 2];  // CTA 0: the partial its peer computed for the long row
  __shared__ int t_slot[TABLE ? 1 : PAIR_MAX_ROWS], t_n[TABLE ? 1 : PAIR_MAX_ROWS];
  __shared__ int s_pair[2];

  cg::cluster_group cluster = cg::this_cluster();
  const int role = blockIdx.x, h = blockIdx.y, i = blockIdx.z, rows = p.rows;
  const int tid = threadIdx.x;
  ATTN_STAMP(0);
  pdl_wait();
  pdl_trigger();

  int r_long, r_short, s_long, s_short, n_long, n_short;
  if constexpr (TABLE) {
    // the step's schedule (built beside the embedding): two entries, no dependent loads
    const int4 a = __ldcg(reinterpret_cast<const int4*>(p.sched) + i);
    const int4 b = __ldcg(reinterpret_cast<const int4*>(p.sched) + (rows - 1 - i));
    r_long = a.x, s_long = a.y, n_long = a.z, r_short = b.x, s_short = b.y, n_short = b.z;
  } else {
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
  ATTN_STAMP(2);
  const bool solo = r_long == r_short;  // the middle row of an odd count
  // keys [cut, n_long) of the long row go to CTA 1 (a multiple of 16 keeps both CTAs' loads aligned to whole groups)
  int cut = n_long;
  if (!solo && n_long - n_short >= 32) cut = min(n_long, ((n_long + n_short) / 2 + 15) & ~15);
  const bool helped = cut < n_long;

  float M, L, O;
  if (role == 0) {
    attend_range<D, SELF>(p, r_long, s_long, h, n_long, 0, cut, true, s_m, s_l, s_acc, M, L, O);
    if (helped) {
      cluster.sync();  // the peer's partial has landed
      if (tid < D) {
        const float pm = s_peer[D], pl = s_peer[D + 1], po = s_peer[tid];
        const float mm = fmaxf(M, pm), w0 = ex2(M - mm), w1 = ex2(pm - mm);
        L = w0 * L + w1 * pl, O = w0 * O + w1 * po;
      }
    }
    if (tid < D) store_out<D>(p, r_long, h, O / L);
  } else {
    if (!solo) {
      attend_range<D, SELF>(p, r_short, s_short, h, n_short, 0, n_short, true, s_m, s_l, s_acc, M, L, O);
      if (tid < D) store_out<D>(p, r_short, h, O / L);
    }
    if (helped) {
      attend_range<D, SELF>(p, r_long, s_long, h, n_long, cut, n_long, false, s_m, s_l, s_acc, M, L, O);
      float* peer = cluster.map_shared_rank(s_peer, 0);
      if (tid < D) peer[tid] = O;
      if (tid == 0) peer[D] = M, peer[D + 1] = L;
      cluster.sync();
    }
  }
  ATTN_STAMP(7);
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

extern "C" {

int64_t b200dec_attention_scratch_floats(int rows, int heads, int head_dim) {
  return (int64_t)rows * heads * MAX_SPLITS * (head_dim + 2);
}

int b200dec_attention(int self, const int32_t* active, const float* q, int ldq, void* kcache, void* vcache,
                      const int32_t* n, int slots, int heads, int head_dim, int cap, float scale, void* out,
                      int out_kind, int rows, float* part, int32_t* count, int32_t* status, int pdl, void* stream) {
  B200_REQUIRE(active && q && kcache && vcache && n && out && status, "attention: null pointer");
  B200_REQUIRE(head_dim == 64 || head_dim == 128, "attention: head_dim %d (64 or 128)", head_dim);
  B200_REQUIRE(rows >= 1 && rows <= 65535 && heads >= 1 && cap >= 1, "attention: rows %d heads %d cap %d", rows,
               heads, cap);
  B200_REQUIRE(ldq % 4 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)kcache & 15) == 0 &&
                   ((uintptr_t)vcache & 15) == 0, "attention: alignment");
  B200_REQUIRE(out_kind == B200DEC_OUT_F16 || out_kind == B200DEC_OUT_F32, "attention: out_kind");
  AttnArgs p{};
  p.active = active, p.q = q, p.k = (__nv_bfloat16*)kcache, p.v = (__nv_bfloat16*)vcache, p.n = n, p.out = out;
  p.part = part, p.count = count, p.status = status;
  p.ldq = ldq, p.H = heads, p.cap = cap, p.slots = slots, p.out_kind = out_kind, p.rows = rows;
  p.splits = (part && count) ? pick_splits(rows, heads, cap) : 1;
  p.scale_log2 = scale * 1.4426950408889634f;
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e;
  if (p.splits == 1 && rows * heads >= 512 && rows <= PAIR_MAX_ROWS) {
    // a large batch: rows paired long with short, two CTAs per pair and head
    const dim3 grid(2, heads, (rows + 1) / 2);
#ifdef B200DEC_TIMELINE
    p.stamps = timeline_next(2 * heads * ((rows + 1) / 2), self ? 3000000 : 4000000);
#endif
    if (head_dim == 64)
      e = self ? launch_kernel(attention_pair_kernel<64, true, false>, grid, dim3(NTHREADS), 0, s, 2, pdl, p)
               : launch_kernel(attention_pair_kernel<64, false, false>, grid, dim3(NTHREADS), 0, s, 2, pdl, p);
    else
      e = self ? launch_kernel(attention_pair_kernel<128, true, false>, grid, dim3(NTHREADS), 0, s, 2, pdl, p)
               : launch_kernel(attention_pair_kernel<128, false, false>, grid, dim3(NTHREADS), 0, s, 2, pdl, p);
    if (e != cudaSuccess) return fail(B200DEC_ECUDA, "attention launch: %s", cudaGetErrorString(e));
    return 0;
  }
  const dim3 grid(heads, rows, p.splits);
#ifdef B200DEC_TIMELINE
  p.stamps = timeline_next(heads * rows * p.splits, self ? 3000000 : 4000000);
#endif
  if (head_dim == 64)
    e = self ? launch_kernel(attention_kernel<64, true>, grid, dim3(NTHREADS), 0, s, 0, pdl, p)
             : launch_kernel(attention_kernel<64, false>, grid, dim3(NTHREADS), 0, s, 0, pdl, p);
  else
    e = self ? launch_kernel(attention_kernel<128, true>, grid, dim3(NTHREADS), 0, s, 0, pdl, p)
             : launch_kernel(attention_kernel<128, false>, grid, dim3(NTHREADS), 0, s, 0, pdl, p);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "attention launch: %s", cudaGetErrorString(e));
  return 0;
}

}  // extern "C"

extern "C" int b200dec_attention_paired(int self, const int32_t* sched, const float* q, int ldq, void* kcache,
                                        void* vcache, int heads, int head_dim, int cap, float scale, void* out,
                                        int out_kind, int rows, int pdl, void* stream) {
  B200_REQUIRE(sched && q && kcache && vcache && out, "attention_paired: null pointer");
  B200_REQUIRE(head_dim == 64 || head_dim == 128, "attention_paired: head_dim %d (64 or 128)", head_dim);
  B200_REQUIRE(rows >= 1 && rows <= PAIR_MAX_ROWS && heads >= 1 && cap >= 1, "attention_paired: rows %d heads %d cap %d",
               rows, heads, cap);
  B200_REQUIRE(ldq % 4 == 0 && ((uintptr_t)q & 15) == 0 && ((uintptr_t)kcache & 15) == 0 &&
                   ((uintptr_t)vcache & 15) == 0 && ((uintptr_t)sched & 15) == 0, "attention_paired: alignment");
  B200_REQUIRE(out_kind == B200DEC_OUT_F16 || out_kind == B200DEC_OUT_F32, "attention_paired: out_kind");
  AttnArgs p{};
  p.sched = sched, p.q = q, p.k = (__nv_bfloat16*)kcache, p.v = (__nv_bfloat16*)vcache, p.out = out;
  p.ldq = ldq, p.H = heads, p.cap = cap, p.out_kind = out_kind, p.rows = rows, p.splits = 1;
  p.scale_log2 = scale * 1.4426950408889634f;
  const dim3 grid(2, heads, (rows + 1) / 2);
#ifdef B200DEC_TIMELINE
  p.stamps = timeline_next(2 * heads * ((rows + 1) / 2), self ? 3000000 : 4000000);
#endif
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e;
  if (head_dim == 64)
    e = self ? launch_kernel(attention_pair_kernel<64, true, true>, grid, dim3(NTHREADS), 0, s, 2, pdl, p)
             : launch_kernel(attention_pair_kernel<64, false, true>, grid, dim3(NTHREADS), 0, s, 2, pdl, p);
  else
    e = self ? launch_kernel(attention_pair_kernel<128, true, true>, grid, dim3(NTHREADS), 0, s, 2, pdl, p)
             : launch_kernel(attention_pair_kernel<128, false, true>, grid, dim3(NTHREADS), 0, s, 2, pdl, p);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "attention_paired launch: %s", cudaGetErrorString(e));
  return 0;
}

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
  return b200dec_attention(self, active, q, ldq, kcache, vcache, n, slots, heads, head_dim, cap, scale, out, out_kind,
                           rows, scratch, count, status, pdl, stream);
}
