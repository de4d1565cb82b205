// Row-wise kernels of the decoding step (embedding + LayerNorm, LayerNorm of the fp32 residual stream, the greedy
// pick and slot bookkeeping, the cross-KV scatter) and the init-time weight packers.
#include "common.cuh"

using namespace b200dec_detail;

namespace b200dec_detail {

char* error_buffer() {
  static thread_local char buf[512] = "";
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "%s: %s", what, cudaGetErrorString(e));
  return 0;
}

}  // namespace b200dec_detail


namespace {

// LayerNorm of a 1024-wide row held by one warp (32 values per lane: chunks of 4 at columns 128 i + 4 lane),
// two-pass fp32 statistics as nn.LayerNorm.
DEVI void ln_row(const float (&v)[32], const float* __restrict__ w, const float* __restrict__ b, float eps, int lane,
                 float (&o)[32]) {
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) s += v[i];
  const float mean = warp_sum(s) * (1.f / D_MODEL);
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float d = v[i] - mean;
    q += d * d;
  }
  const float rstd = rsqrtf(warp_sum(q) * (1.f / D_MODEL) + eps);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = i * 128 + lane * 4;
    const float4 ww = *reinterpret_cast<const float4*>(w + c), bb = *reinterpret_cast<const float4*>(b + c);
    o[4 * i] = (v[4 * i] - mean) * rstd * ww.x + bb.x;
    o[4 * i + 1] = (v[4 * i + 1] - mean) * rstd * ww.y + bb.y;
    o[4 * i + 2] = (v[4 * i + 2] - mean) * rstd * ww.z + bb.z;
    o[4 * i + 3] = (v[4 * i + 3] - mean) * rstd * ww.w + bb.w;
  }
}

DEVI void store_row(const float (&o)[32], void* dst, int kind, size_t row, int lane) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = i * 128 + lane * 4;
    if (kind == B200DEC_OUT_F16)
      *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(dst) + row * D_MODEL + c) =
          make_uint2(pack_f16(o[4 * i], o[4 * i + 1]), pack_f16(o[4 * i + 2], o[4 * i + 3]));
    else
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + row * D_MODEL + c) =
          make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
  }
}

// ---- row schedule: the step's rows ranked by decreasing length, once per step -------------------------------------
// The paired attention kernel gives the i-th longest row and the i-th shortest to one cluster; the ranking is the same
// for all layers of a step, so one CTA computes it at the start of the step (beside the embedding) and the sixteen
// attention launches read two table entries each. Entry i = {row, slot, length, 0} of the row of rank i.
constexpr int SCHED_MAX_ROWS = 256;
struct SchedArgs {
  const int* active;
  const int* pos;        // per slot: keys in the self cache (the new token's position)
  const int* cross_len;  // per slot: encoder frames
  int* sched_self;       // (rows, 4) or null
  int* sched_cross;
  int* status;
  int slots, seq, frames, rows;
  int prefetch_keys;     // most keys (over all rows of a table) marked for prefetch into L2; 0: none
};

DEVI void rank_rows(const SchedArgs& p, const int* len, bool self, int* out, int* t_s, int* t_n) {
  const int cap = self ? p.seq : p.frames;
  __shared__ int s_total;
  if (threadIdx.x == 0) s_total = 0;
  __syncthreads();
  for (int r = threadIdx.x; r < p.rows; r += blockDim.x) {
    int s = p.active[r];
    if (s < 0 || s > p.slots) {
      atomicOr(p.status, B200DEC_ST_SLOT_RANGE);
      s = p.slots;
    }
    int n = len[s];
    if (self ? (n < 0 || n >= cap) : (n < 1 || n > cap)) {
      atomicOr(p.status, self ? B200DEC_ST_POS_RANGE : B200DEC_ST_FRAMES_RANGE);
      n = self ? max(0, min(n, cap - 1)) : max(1, min(n, cap));
    }
    t_s[r] = s, t_n[r] = n;
    atomicAdd(&s_total, n);
  }
  __syncthreads();
  const int total = s_total;
  for (int r = threadIdx.x; r < p.rows; r += blockDim.x) {
    const int n = t_n[r];
    int rank = 0;
    for (int j = 0; j < p.rows; ++j) rank += (t_n[j] > n) || (t_n[j] == n && j < r);  // ties by row
    // the row's share of the prefetch budget: all its keys when the launch fits, else in proportion (whole 1 KB runs)
    int pf = 0;
    if (p.prefetch_keys > 0)
      pf = total <= p.prefetch_keys ? n : (int)((long long)n * p.prefetch_keys / total) & ~7;
    *reinterpret_cast<int4*>(out + 4 * rank) = make_int4(r, t_s[r], n, pf);
  }
  __syncthreads();
}

DEVI void build_schedules(const SchedArgs& p) {
  __shared__ int t_s[SCHED_MAX_ROWS], t_n[SCHED_MAX_ROWS];
  if (p.sched_self) rank_rows(p, p.pos, true, p.sched_self, t_s, t_n);
  if (p.sched_cross) rank_rows(p, p.cross_len, false, p.sched_cross, t_s, t_n);
}

__global__ void __launch_bounds__(128) row_schedule_kernel(const SchedArgs p) {
  pdl_wait();
  pdl_trigger();
  build_schedules(p);
}

// o (a row in registers) -> fp16(o * gamma) and the row's (sum, sum of squares): the ready operand of a
// LayerNorm-folding projection and the statistics that go with it (one slot per row)
DEVI void ln_operand_row(const float (&o)[32], const float* gamma, void* dst, float* stats, size_t row, int lane) {
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = i * 128 + lane * 4;
    const float4 g = *reinterpret_cast<const float4*>(gamma + c);
    *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(dst) + row * D_MODEL + c) =
        make_uint2(pack_f16(o[4 * i] * g.x, o[4 * i + 1] * g.y), pack_f16(o[4 * i + 2] * g.z, o[4 * i + 3] * g.w));
    s1 += (o[4 * i] + o[4 * i + 1]) + (o[4 * i + 2] + o[4 * i + 3]);
    s2 += (o[4 * i] * o[4 * i] + o[4 * i + 1] * o[4 * i + 1]) + (o[4 * i + 2] * o[4 * i + 2] + o[4 * i + 3] * o[4 * i + 3]);
  }
  s1 = warp_sum(s1), s2 = warp_sum(s2);
  if (lane == 0) reinterpret_cast<float2*>(stats)[row] = make_float2(s1, s2);
}

struct EmbedArgs {
  SchedArgs sched;  // sched.rows == 0: no schedule; else the grid's last CTA builds it
  const int* active;
  const int64_t* tok;
  const int* pos;
  const __nv_bfloat16* embed;
  const __nv_bfloat16* ptab;
  b200dec_norm ln0, ln1;
  float* x;
  void* x16;  // null, or (rows, 1024) fp16 = x * next_gamma with the rows' (sum, sum of squares) in stats (rows, 2):
  const float* next_gamma;  // the ready operand of the first LayerNorm-folding projection
  float* stats;
  void* hn;
  int* status;
  int vocab, max_pos, slots, hn_kind, rows;
};

__global__ void __launch_bounds__(128) embed_ln_kernel(const EmbedArgs p) {
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  pdl_wait();     // a dependent grid may start only after this one has seen its predecessor complete, so what a
  pdl_trigger();  // kernel reads before its own wait was written at least two kernels earlier
  if (p.sched.rows > 0 && blockIdx.x == gridDim.x - 1) {  // the extra CTA
    build_schedules(p.sched);
    return;
  }
  if (row >= p.rows) return;
  int s = p.active[row];
  if (s < 0 || s > p.slots) {
    if (lane == 0) atomicOr(p.status, B200DEC_ST_SLOT_RANGE);
    s = p.slots;
  }
  int64_t t = p.tok[s];
  int ps = p.pos[s];
  if (t < 0 || t >= p.vocab) {
    if (lane == 0) atomicOr(p.status, B200DEC_ST_TOKEN_RANGE);
    t = 0;
  }
  if (ps < 0 || ps >= p.max_pos) {
    if (lane == 0) atomicOr(p.status, B200DEC_ST_POS_RANGE);
    ps = 0;
  }
  float v[32], o[32];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = i * 128 + lane * 4;
    const uint2 e = *reinterpret_cast<const uint2*>(p.embed + (size_t)t * D_MODEL + c);
    const uint2 q = *reinterpret_cast<const uint2*>(p.ptab + (size_t)ps * D_MODEL + c);
    v[4 * i] = bf16_lo(e.x) + bf16_lo(q.x), v[4 * i + 1] = bf16_hi(e.x) + bf16_hi(q.x);
    v[4 * i + 2] = bf16_lo(e.y) + bf16_lo(q.y), v[4 * i + 3] = bf16_hi(e.y) + bf16_hi(q.y);
  }
  ln_row(v, p.ln0.w, p.ln0.b, p.ln0.eps, lane, o);
  store_row(o, p.x, B200DEC_OUT_F32, row, lane);
  if (p.x16) ln_operand_row(o, p.next_gamma, p.x16, p.stats, row, lane);  // what the first projection stages
  if (p.hn) {  // optionally also the first layer's LayerNorm of the new row
    ln_row(o, p.ln1.w, p.ln1.b, p.ln1.eps, lane, v);
    store_row(v, p.hn, p.hn_kind, row, lane);
  }
}

struct LnArgs {
  const float* x;
  b200dec_norm ln;
  void* hn;
  int hn_kind, rows;
};

__global__ void __launch_bounds__(128) layer_norm_kernel(const LnArgs p) {
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  pdl_wait();     // a dependent grid may start only after this one has seen its predecessor complete, so what a
  pdl_trigger();  // kernel reads before its own wait was written at least two kernels earlier
  if (row >= p.rows) return;
  float v[32], o[32];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float4 a = ld_cg_f4(p.x + (size_t)row * D_MODEL + i * 128 + lane * 4);
    v[4 * i] = a.x, v[4 * i + 1] = a.y, v[4 * i + 2] = a.z, v[4 * i + 3] = a.w;
  }
  ln_row(v, p.ln.w, p.ln.b, p.ln.eps, lane, o);
  store_row(o, p.hn, p.hn_kind, row, lane);
}

__global__ void __launch_bounds__(128) ln_rows16_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                        int rows, void* out16, float* stats) {
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  float v[32];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float4 a = ld_cg_f4(x + (size_t)row * D_MODEL + i * 128 + lane * 4);
    v[4 * i] = a.x, v[4 * i + 1] = a.y, v[4 * i + 2] = a.z, v[4 * i + 3] = a.w;
  }
  ln_operand_row(v, gamma, out16, stats, row, lane);
}

struct PickArgs {
  const float* part_max;
  const int* part_idx;
  const int* active;
  int64_t* tok;
  int* pos;
  uint8_t* finished;
  const int64_t* forced;
  const int* plen;
  const int* limit;
  int64_t* out;
  int64_t* argmax;
  uint8_t* flags_host;  // pinned host memory mapped into the device's address space, or null: a row that ends sets
                        // its slot's byte there (one posted write over the bus per ending row: the step waits for
                        // no copy); the host clears the byte when it admits into the slot
  int partials, rows, dummy, max_prompt, out_cols, eos;
};

// one warp per row: first index of the maximum over the row's partials, then dec_pick's bookkeeping
__global__ void __launch_bounds__(128) pick_kernel(const PickArgs p) {
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  pdl_wait();     // a dependent grid may start only after this one has seen its predecessor complete, so what a
  pdl_trigger();  // kernel reads before its own wait was written at least two kernels earlier
  if (row >= p.rows) return;
  const int s = p.active[row];
  if (s < 0 || s >= p.dummy) return;  // the dummy slot (and anything outside the table) never advances
  float best = -INFINITY;
  int arg = 0x7fffffff;
  for (int i = lane; i < p.partials; i += 32) {
    const float v = __ldcg(p.part_max + (size_t)row * p.partials + i);
    const int a = __ldcg(p.part_idx + (size_t)row * p.partials + i);
    if (v > best || (v == best && a < arg)) best = v, arg = a;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
    if (ob > best || (ob == best && oa < arg)) best = ob, arg = oa;
  }
  if (lane != 0) return;
  if (arg == 0x7fffffff) arg = 0;  // a row of NaN
  if (p.argmax) p.argmax[s] = arg;
  if (p.finished[s]) return;  // ended at an earlier step: nothing moves until the host retires the slot
  const int at = p.pos[s] + 1;
  const bool in_prompt = at < p.plen[s];
  const int64_t nt = in_prompt ? p.forced[(size_t)s * p.max_prompt + min(at, p.max_prompt - 1)] : (int64_t)arg;
  if (at < p.out_cols) p.out[(size_t)s * p.out_cols + at] = nt;
  p.tok[s] = nt;
  p.pos[s] = at;
  const uint8_t done = (!in_prompt && (nt == p.eos || at >= p.limit[s])) ? 1 : 0;
  p.finished[s] = done;
  if (done && p.flags_host) p.flags_host[s] = 1;
}

// A measurement aid, not a step of the decoder: every CTA reads its own contiguous run of `chunk16` 16-byte pieces with
// the attention kernels' loads (streaming, 8 in flight per thread) and does nothing else. What it reaches is the
// speed a launch of that grid and that many bytes can read at all, ramp-up and tail included.
struct ProbeArgs {
  const uint4* src;
  size_t chunk16;
  uint32_t* sink;
};

__global__ void __launch_bounds__(128) read_probe_kernel(const ProbeArgs a) {
  constexpr int U = 8;
  pdl_wait();
  const uint4* p = a.src + (size_t)blockIdx.x * a.chunk16;
  const size_t chunk16 = a.chunk16;
  uint32_t* sink = a.sink;
  uint32_t acc = 0;
  for (size_t i = threadIdx.x; i < chunk16; i += 128 * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = i + u * 128 < chunk16 ? ld_stream16(p + i + u * 128) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int u = 0; u < U; ++u) acc += (v[u].x ^ v[u].y) + (v[u].z ^ v[u].w);
  }
  pdl_trigger();
  if (acc == 0x9e3779b9u && sink) *sink = acc;  // keeps the loads alive; practically never taken
}

// kv (nrows, L * 2 * H * D) fp32 -> bf16 caches (L, S1, H, T, D); one thread per 8 values
__global__ void scatter_kv_kernel(const float* __restrict__ kv, const int* __restrict__ slot_of,
                                  const int* __restrict__ frame_of, __nv_bfloat16* ck, __nv_bfloat16* cv, int nrows,
                                  int L, int S1, int H, int D, int T) {
  const int d8n = D / 8, chunks = L * 2 * H * d8n;
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)nrows * chunks) return;
  const int row = idx / chunks, c = idx % chunks;
  const int d8 = c % d8n, h = (c / d8n) % H, kvi = (c / (d8n * H)) % 2, l = c / (d8n * H * 2);
  const int slot = slot_of[row], frame = frame_of[row];
  if (slot < 0 || slot >= S1 || frame < 0 || frame >= T) return;
  const float* src = kv + (size_t)row * chunks * 8 + (size_t)c * 8;
  const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
  __nv_bfloat16* dst = (kvi ? cv : ck) + ((((size_t)l * S1 + slot) * H + h) * T + frame) * D + d8 * 8;
  *reinterpret_cast<uint4*>(dst) =
      make_uint4(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w), pack_bf16(b.x, b.y), pack_bf16(b.z, b.w));
}

// The same into int8 caches with one fp32 scale per head vector (the reference's int8 mode, kernels/csrc/
// decoder_ops.cu:176-204): the values are rounded to bf16 first (what the bf16 cache would hold), then
// scale = absmax / 127 (1 for a zero vector), q = rint(clamp(x * (1 / scale), +-127)). D / 8 threads per vector.
__global__ void scatter_kv_q8_kernel(const float* __restrict__ kv, const int* __restrict__ slot_of,
                                     const int* __restrict__ frame_of, int8_t* ck, int8_t* cv, float* cks, float* cvs,
                                     int nrows, int L, int S1, int H, int D, int T) {
  const int d8n = D / 8, chunks = L * 2 * H * d8n;  // d8n = 8 or 16 threads per vector, aligned inside a warp
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = idx < (size_t)nrows * chunks;
  const int row = live ? idx / chunks : 0, c = live ? idx % chunks : 0;
  const int d8 = c % d8n, h = (c / d8n) % H, kvi = (c / (d8n * H)) % 2, l = c / (d8n * H * 2);
  float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (live) {
    const float* src = kv + (size_t)row * chunks * 8 + (size_t)c * 8;
    const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 4);
    const uint32_t w[4] = {pack_bf16(a.x, a.y), pack_bf16(a.z, a.w), pack_bf16(b.x, b.y), pack_bf16(b.z, b.w)};
#pragma unroll
    for (int i = 0; i < 4; ++i) f[2 * i] = bf16_lo(w[i]), f[2 * i + 1] = bf16_hi(w[i]);
  }
  float mx = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) mx = fmaxf(mx, fabsf(f[i]));
  for (int o = 1; o < d8n; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (!live) return;
  const int slot = slot_of[row], frame = frame_of[row];
  if (slot < 0 || slot >= S1 || frame < 0 || frame >= T) return;
  const float sc = mx > 0.f ? __fdiv_rn(mx, 127.f) : 1.f, inv = __fdiv_rn(1.f, sc);
  uint32_t w[2] = {0, 0};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int q = __float2int_rn(fminf(fmaxf(__fmul_rn(f[i], inv), -127.f), 127.f));
    w[i >> 2] |= (uint32_t)(q & 0xff) << ((i & 3) * 8);
  }
  const size_t vec = (((size_t)l * S1 + slot) * H + h) * T + frame;
  *reinterpret_cast<uint2*>((kvi ? cv : ck) + vec * D + d8 * 8) = make_uint2(w[0], w[1]);
  if (d8 == 0) (kvi ? cvs : cks)[vec] = sc;
}

// ---- packers -------------------------------------------------------------------------------------------------------

__constant__ int c_w8_perm[16] = {0, 1, 8, 9, 2, 3, 10, 11, 4, 5, 12, 13, 6, 7, 14, 15};

// one CTA per row: scale = max(absmax, 1e-12) / 127; q = clamp(rint(w / scale)); the division is IEEE fp32 (as
// torch's), not a multiplication by the reciprocal. layout 0: int8 (n, k); 1: uint8 + 128 with W8_PERM.
__global__ void __launch_bounds__(256) quantize_rows_kernel(const float* __restrict__ w, int k, void* q,
                                                            float* __restrict__ scale, int layout) {
  __shared__ float red[8];
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* wr = w + (size_t)row * k;
  float mx = 0.f;
  for (int i = tid; i < k; i += 256) mx = fmaxf(mx, fabsf(wr[i]));
#pragma unroll
  for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) mx = fmaxf(mx, red[i]);
  const float s = __fdiv_rn(fmaxf(mx, 1e-12f), 127.f);
  if (tid == 0) scale[row] = s;
  for (int i = tid; i < k; i += 256) {
    const float v = fminf(fmaxf(rintf(__fdiv_rn(wr[i], s)), -127.f), 127.f);
    if (layout == 0) {
      reinterpret_cast<int8_t*>(q)[(size_t)row * k + i] = (int8_t)v;
    } else {
      // output byte j of a 16-group takes input byte W8_PERM[j]: scatter input i to the j with PERM[j] == i
      const int gi = i & 15;
      int j = 0;
#pragma unroll
      for (int t = 0; t < 16; ++t)
        if (c_w8_perm[t] == gi) j = t;
      reinterpret_cast<uint8_t*>(q)[(size_t)row * k + (i & ~15) + j] = (uint8_t)((int)v + 128);
    }
  }
}

// one thread per group of four: zero the two smallest magnitudes, the lower index first on ties
__global__ void prune24_kernel(const float* __restrict__ w, float* __restrict__ out, size_t groups) {
  const size_t gidx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gidx >= groups) return;
  const float4 v = *reinterpret_cast<const float4*>(w + gidx * 4);
  float a[4] = {v.x, v.y, v.z, v.w};
  const float m[4] = {fabsf(v.x), fabsf(v.y), fabsf(v.z), fabsf(v.w)};
  // rank of element i in a stable ascending sort of the magnitudes
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int rank = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) rank += (m[j] < m[i]) || (m[j] == m[i] && j < i);
    if (rank < 2) a[i] = 0.f;
  }
  *reinterpret_cast<float4*>(out + gidx * 4) = make_float4(a[0], a[1], a[2], a[3]);
}

// one thread per selector word (8 groups of four = 32 values of a row)
__global__ void compress24_kernel(const int8_t* __restrict__ q, int n, int k, int8_t* __restrict__ kept,
                                  uint32_t* __restrict__ words, int* bad) {
  const size_t widx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int wpr = k / 32;
  if (widx >= (size_t)n * wpr) return;
  const int row = widx / wpr, wc = widx % wpr;
  const int8_t* src = q + (size_t)row * k + wc * 32;
  int8_t* dst = kept + (size_t)row * (k / 2) + wc * 16;
  uint32_t word = 0;
  for (int gi = 0; gi < 8; ++gi) {
    const int8_t v[4] = {src[gi * 4], src[gi * 4 + 1], src[gi * 4 + 2], src[gi * 4 + 3]};
    // kept positions: the nonzero ones, made up with the lowest zero positions, in increasing order
    int nz = 0;
    for (int i = 0; i < 4; ++i) nz += v[i] != 0;
    if (nz > 2) atomicExch(bad, 1);
    int need_zero = nz >= 2 ? 0 : 2 - nz, cnt = 0, keep[2] = {0, 1};
    for (int i = 0; i < 4 && cnt < 2; ++i) {
      if (v[i] != 0) {
        keep[cnt++] = i;
      } else if (need_zero > 0) {
        keep[cnt++] = i;
        --need_zero;
      }
    }
    dst[gi * 2] = v[keep[0]];
    dst[gi * 2 + 1] = v[keep[1]];
    word |= (uint32_t)(keep[0] | (keep[1] << 2)) << (4 * gi);
  }
  words[widx] = word;
}

}  // namespace

namespace b200dec_detail {

int embed_ln_impl(const int32_t* active, const int64_t* tok, const int32_t* pos, const void* embed,
                  const void* pos_table, int vocab, int max_pos, int slots, b200dec_norm ln0, b200dec_norm ln1, float* x,
                  void* hn, int hn_kind, int rows, int32_t* status, int pdl, void* stream, const int32_t* cross_len,
                  int seq, int frames, int32_t* sched_self, int32_t* sched_cross, void* x16, const float* next_gamma,
                  float* stats, int prefetch_keys) {
  B200_REQUIRE(active && tok && pos && embed && pos_table && x && status && ln0.w && ln0.b && (!hn || (ln1.w && ln1.b)),
               "embed_ln: null pointer");
  B200_REQUIRE(rows >= 1, "embed_ln: rows %d", rows);
  B200_REQUIRE(!x16 || (next_gamma && stats), "embed_ln: the fp16 operand needs the next gamma and a place for the sums");
  const bool sched = (sched_self || sched_cross) && rows <= SCHED_MAX_ROWS;
  B200_REQUIRE(!sched || !sched_cross || cross_len, "embed_ln: a cross schedule needs the frame counts");
  EmbedArgs p{SchedArgs{active, pos, cross_len, sched_self, sched_cross, status, slots, seq, frames, sched ? rows : 0,
                        prefetch_keys},
              active, tok, pos, (const __nv_bfloat16*)embed, (const __nv_bfloat16*)pos_table, ln0, ln1, x, x16, next_gamma,
              stats, hn, status, vocab, max_pos, slots, hn_kind, rows};
  const cudaError_t e = launch_kernel(embed_ln_kernel, dim3((rows + 3) / 4 + (sched ? 1 : 0)), dim3(128), 0,
                                      (cudaStream_t)stream, 0, pdl, p);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "embed_ln launch: %s", cudaGetErrorString(e));
  return 0;
}

int layer_norm_impl(const float* x, b200dec_norm ln, void* hn, int hn_kind, int rows, int pdl, void* stream) {
  B200_REQUIRE(x && hn && ln.w && ln.b && rows >= 1, "layer_norm: bad arguments");
  LnArgs p{x, ln, hn, hn_kind, rows};
  const cudaError_t e = launch_kernel(layer_norm_kernel, dim3((rows + 3) / 4), dim3(128), 0, (cudaStream_t)stream, 0,
                                      pdl, p);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "layer_norm launch: %s", cudaGetErrorString(e));
  return 0;
}

int pick_impl(const float* part_max, const int32_t* part_idx, int partials, const int32_t* active, int rows, int dummy,
              int64_t* tok, int32_t* pos, uint8_t* finished, const int64_t* forced, int max_prompt,
              const int32_t* plen, const int32_t* limit, int64_t* out, int out_cols, int eos, int64_t* argmax,
              uint8_t* flags_host, int pdl, void* stream) {
  B200_REQUIRE(part_max && part_idx && active && tok && pos && finished && forced && plen && limit && out,
               "pick: null pointer");
  B200_REQUIRE(rows >= 1 && partials >= 1 && max_prompt >= 1, "pick: sizes");
  PickArgs p{part_max, part_idx, active, tok, pos, finished, forced, plen, limit, out, argmax, flags_host,
             partials, rows, dummy, max_prompt, out_cols, eos};
  const cudaError_t e = launch_kernel(pick_kernel, dim3((rows + 3) / 4), dim3(128), 0, (cudaStream_t)stream, 0, pdl, p);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "pick launch: %s", cudaGetErrorString(e));
  return 0;
}

}  // namespace b200dec_detail

extern "C" {

const char* b200dec_last_error(void) { return error_buffer(); }
int b200dec_version(void) { return 1; }

int b200dec_embed_ln(const int32_t* active, const int64_t* tok, const int32_t* pos, const void* embed,
                     const void* pos_table, int vocab, int max_pos, int slots, b200dec_norm ln0, b200dec_norm ln1,
                     float* x, void* hn, int hn_kind, int rows, int32_t* status, int pdl, void* stream) {
  return embed_ln_impl(active, tok, pos, embed, pos_table, vocab, max_pos, slots, ln0, ln1, x, hn, hn_kind, rows, status,
                       pdl, stream, nullptr, 0, 0, nullptr, nullptr, nullptr, nullptr, nullptr, 0);
}

int b200dec_ln_rows16(const float* x, const float* gamma, int rows, void* out16, float* stats, void* stream) {
  B200_REQUIRE(x && gamma && out16 && stats && rows >= 1 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out16 & 7) == 0,
               "ln_rows16: bad arguments");
  ln_rows16_kernel<<<(rows + 3) / 4, 128, 0, (cudaStream_t)stream>>>(x, gamma, rows, out16, stats);
  return check_launch("ln_rows16");
}

int b200dec_row_schedule(const int32_t* active, const int32_t* pos, const int32_t* cross_len, int slots, int seq,
                         int frames, int rows, int prefetch_keys, int32_t* sched_self, int32_t* sched_cross,
                         int32_t* status, void* stream) {
  B200_REQUIRE(active && status && (sched_self || sched_cross), "row_schedule: null pointer");
  B200_REQUIRE((!sched_self || pos) && (!sched_cross || cross_len), "row_schedule: a table without its lengths");
  B200_REQUIRE(rows >= 1 && rows <= SCHED_MAX_ROWS, "row_schedule: rows %d (1..%d)", rows, SCHED_MAX_ROWS);
  B200_REQUIRE(prefetch_keys >= 0, "row_schedule: prefetch_keys %d", prefetch_keys);
  SchedArgs p{active, pos, cross_len, sched_self, sched_cross, status, slots, seq, frames, rows, prefetch_keys};
  const cudaError_t e = launch_kernel(row_schedule_kernel, dim3(1), dim3(128), 0, (cudaStream_t)stream, 0, 0, p);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "row_schedule launch: %s", cudaGetErrorString(e));
  return 0;
}

int b200dec_layer_norm(const float* x, b200dec_norm ln, void* hn, int hn_kind, int rows, int pdl, void* stream) {
  return layer_norm_impl(x, ln, hn, hn_kind, rows, pdl, stream);
}

int b200dec_pick(const float* part_max, const int32_t* part_idx, int partials, const int32_t* active, int rows,
                 int dummy, int64_t* tok, int32_t* pos, uint8_t* finished, const int64_t* forced, int max_prompt,
                 const int32_t* plen, const int32_t* limit, int64_t* out, int out_cols, int eos, int64_t* argmax,
                 uint8_t* flags_host, int pdl, void* stream) {
  return pick_impl(part_max, part_idx, partials, active, rows, dummy, tok, pos, finished, forced, max_prompt, plen,
                   limit, out, out_cols, eos, argmax, flags_host, pdl, stream);
}

int b200dec_scatter_kv(const float* kv, const int32_t* slot_of, const int32_t* frame_of, void* ck, void* cv,
                       int nrows, int layers, int slots_plus_1, int heads, int head_dim, int frames, void* stream) {
  B200_REQUIRE(kv && slot_of && frame_of && ck && cv, "scatter_kv: null pointer");
  B200_REQUIRE(head_dim % 8 == 0 && nrows >= 0, "scatter_kv: head_dim %d", head_dim);
  if (nrows == 0) return 0;
  const size_t total = (size_t)nrows * layers * 2 * heads * (head_dim / 8);
  scatter_kv_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      kv, slot_of, frame_of, (__nv_bfloat16*)ck, (__nv_bfloat16*)cv, nrows, layers, slots_plus_1, heads, head_dim,
      frames);
  return check_launch("scatter_kv");
}

int b200dec_read_probe(const void* src, int ctas, int64_t bytes_per_cta, int32_t* sink, int pdl, void* stream) {
  B200_REQUIRE(src && ((uintptr_t)src & 15) == 0, "read_probe: src must be 16-byte aligned");
  B200_REQUIRE(ctas >= 1 && ctas <= 65535 * 16 && bytes_per_cta >= 16 && bytes_per_cta % 16 == 0,
               "read_probe: ctas %d, bytes_per_cta %lld (a multiple of 16)", ctas, (long long)bytes_per_cta);
  const ProbeArgs a{reinterpret_cast<const uint4*>(src), (size_t)(bytes_per_cta / 16), reinterpret_cast<uint32_t*>(sink)};
  const cudaError_t e = launch_kernel(read_probe_kernel, dim3(ctas), dim3(128), 0, (cudaStream_t)stream, 0, pdl != 0, a);
  if (e != cudaSuccess) return fail(B200DEC_ECUDA, "read_probe launch: %s", cudaGetErrorString(e));
  return 0;
}

int b200dec_scatter_kv_q8(const float* kv, const int32_t* slot_of, const int32_t* frame_of, void* ck, void* cv,
                          float* ck_scale, float* cv_scale, int nrows, int layers, int slots_plus_1, int heads,
                          int head_dim, int frames, void* stream) {
  B200_REQUIRE(kv && slot_of && frame_of && ck && cv && ck_scale && cv_scale, "scatter_kv_q8: null pointer");
  B200_REQUIRE((head_dim == 64 || head_dim == 128) && nrows >= 0, "scatter_kv_q8: head_dim %d (64 or 128)", head_dim);
  if (nrows == 0) return 0;
  const size_t total = (size_t)nrows * layers * 2 * heads * (head_dim / 8);  // a multiple of 8 or 16: whole vectors
  scatter_kv_q8_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      kv, slot_of, frame_of, (int8_t*)ck, (int8_t*)cv, ck_scale, cv_scale, nrows, layers, slots_plus_1, heads, head_dim,
      frames);
  return check_launch("scatter_kv_q8");
}

int b200dec_quantize_rows(const float* w, int n, int k, int8_t* q, float* scale, void* stream) {
  B200_REQUIRE(w && q && scale && n >= 1 && k >= 1, "quantize_rows: bad arguments");
  quantize_rows_kernel<<<n, 256, 0, (cudaStream_t)stream>>>(w, k, q, scale, 0);
  return check_launch("quantize_rows");
}

int b200dec_prepare_w8(const float* w, int n, int k, uint8_t* u8, float* scale, void* stream) {
  B200_REQUIRE(w && u8 && scale && n >= 1 && k % 16 == 0, "prepare_w8: K must be a multiple of 16");
  quantize_rows_kernel<<<n, 256, 0, (cudaStream_t)stream>>>(w, k, u8, scale, 1);
  return check_launch("prepare_w8");
}

int b200dec_prune24(const float* w, int n, int k, float* out, void* stream) {
  B200_REQUIRE(w && out && k % 4 == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)out & 15) == 0, "prune24: shape");
  const size_t groups = (size_t)n * k / 4;
  prune24_kernel<<<(unsigned)((groups + 255) / 256), 256, 0, (cudaStream_t)stream>>>(w, out, groups);
  return check_launch("prune24");
}

int b200dec_compress24(const int8_t* q, int n, int k, int8_t* kept, int32_t* words, int32_t* bad, void* stream) {
  B200_REQUIRE(q && kept && words && bad && k % 32 == 0, "compress24: K must be a multiple of 32");
  const size_t total = (size_t)n * (k / 32);
  compress24_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(q, n, k, kept,
                                                                                       (uint32_t*)words, bad);
  return check_launch("compress24");
}

}  // extern "C"
