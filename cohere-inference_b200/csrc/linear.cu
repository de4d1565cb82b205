// Small-M projections of the decoding step: out (rows, N) = act(A (rows, K) x W^T * scale + bias), rows <= 128.
//
// A step's projections are bound by reading their weights once from HBM, each one is tiny (1 - 16 MB), and fifty of
// them run back to back, so the kernel (linear_kernel.cuh) is built for low latency per launch:
//   * Weights are the M operand of mma.sync m16n8k16 ("swap A/B": 16 output channels x the step's rows), so a warp
//     owns 16 channels and streams exactly their bytes. They are re-tiled once (tile_* kernels below) so that every
//     warp-wide 16-byte load is one contiguous 512-byte run and the bytes land in registers already in fragment
//     order: nothing goes through shared memory, and all loads of a warp's K slice are issued up front, before the
//     kernel waits for its predecessor (programmatic dependent launch), so they overlap the previous kernel's tail.
//   * K is split over the CTAs of a thread-block cluster and N over grid.y, so even a 1024 x 1024 matrix spreads over
//     128 SMs. Each CTA pushes its partial tile into the shared memory of the CTA that owns those channels
//     (distributed shared memory stores), one cluster barrier, then every CTA adds the slices of its channels in rank
//     order (deterministic, no workspace, no atomics) and applies the fused epilogue: scale, bias, activation, and
//     either a store (fp16 / fp32), an add into the fp32 residual stream, or the per-tile argmax of the vocabulary
//     projection.
//   * LayerNorm is folded into the projection that consumes it, so the step has no normalisation kernels and no
//     extra barrier: with a per-row shift c the kernel multiplies (x - c) * gamma, each CTA also sums its slice's
//     (x - c) and (x - c)^2 and pushes them along with its partial tile, and the finishing CTA applies
//     y = rstd * (acc * scale - (mean - c) * g) + b', an exact rewriting of LayerNorm(x) W^T + b with
//     g[n] = sum_k gamma[k] W[n][k] and b'[n] = b[n] + sum_k beta[k] W[n][k] precomputed per output channel.
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
#include "linear_kernel.cuh"

using namespace b200dec_detail;

namespace {

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

bool fits_any(int kind, bool split, int ln, int warps, int k, int ksplit, int rows) {
  switch (kind) {
    case B200DEC_W_INT8: return fits_int8(split, ln, warps, k, ksplit, rows);
    case B200DEC_W_BF16: return fits_bf16(split, ln, warps, k, ksplit, rows);
    case B200DEC_W_INT8_24: return fits_24(split, ln, warps, k, ksplit, rows);
    case B200DEC_W_F16: return fits_f16(split, ln, warps, k, ksplit, rows);
    case B200DEC_W_INT8_UMMA:  // linear_umma.cu: fp16 rows, plain or as a LayerNorm's ready operand
    case B200DEC_W_F16_UMMA:
    case B200DEC_W_INT8_24_UMMA:
      return !split && rows <= 128 && ln != 1 &&
             ((k == D_MODEL && (ksplit == 4 || ksplit == 8)) || (k == 4 * D_MODEL && ksplit == 8 && ln == 0));
  }
  return false;
}

}  // namespace
namespace b200dec_detail {
int linear_umma_impl(const b200dec_weight* w, const void* a, int a_kind, const b200dec_norm* ln, int lda, int rows,
                     void* out, int out_kind, int ldo, int act, const b200dec_ln_link* link, int32_t* status, int pdl,
                     void* stream);
}
namespace {

int run_linear(const b200dec_weight* w, const void* a, int a_kind, const b200dec_norm* ln, int lda, int rows, void* out,
               int out_kind, int ldo, int act, float* pmax, int* pidx, float* logits, int head, int pdl, void* stream,
               const b200dec_ln_link* link = nullptr, const KvPrefetch* pf = nullptr) {
  B200_REQUIRE(w && w->w && a, "linear: null pointer");
  B200_REQUIRE(rows >= 1 && rows <= 128, "linear: rows %d outside 1..128", rows);
  if (is_umma_kind(w->kind)) {  // the tcgen05 kernel of linear_umma.cu
    B200_REQUIRE(!head && link && link->status, "linear: a tcgen05 projection goes through b200dec_linear_linked with a "
                 "status word");
    return linear_umma_impl(w, a, a_kind, ln, lda, rows, out, out_kind, ldo, act, link, link->status, pdl, stream);
  }
  B200_REQUIRE(w->warps == 4 || w->warps == 8, "linear: warps must be 4 or 8");
  B200_REQUIRE(w->ksplit == 1 || w->ksplit == 2 || w->ksplit == 4 || w->ksplit == 8, "linear: ksplit %d", w->ksplit);
  B200_REQUIRE(w->n % (16 * w->warps) == 0 && w->k % w->ksplit == 0, "linear: shape (%d, %d) vs tile", w->n, w->k);
  B200_REQUIRE((16 * w->warps) % (8 * w->ksplit) == 0, "linear: warps %d too few for ksplit %d", w->warps, w->ksplit);
  B200_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)w->w & 15) == 0, "linear: operands must be 16-byte aligned");
  B200_REQUIRE(lda % 8 == 0 && lda >= w->k, "linear: lda %d", lda);
  B200_REQUIRE((w->kind == B200DEC_W_BF16 || w->kind == B200DEC_W_F16) == (w->scale == nullptr),
               "linear: scale present iff int8");
  const bool split = a_kind == B200DEC_A_F32_SPLIT;
  B200_REQUIRE(split || a_kind == B200DEC_A_F16 || a_kind == B200DEC_A_F16_ROWS16, "linear: a_kind %d", a_kind);
  // 0: no LayerNorm; 1: folded, the rows are fp32; 2: folded, the rows are fp16 copies of the LayerNorm's input
  int lnorm = ln == nullptr ? 0 : a_kind == B200DEC_A_F16_ROWS16 ? 2 : 1;
  if (lnorm == 2 && !fits_any(w->kind, false, 2, w->warps, w->k, w->ksplit, rows < 64 ? rows : 64))
    return fail(B200DEC_EINVAL, "linear: fp16 LayerNorm rows need int8 weights and a K slice of at most 256");
  const b200dec_ln_link none{};
  const b200dec_ln_link lk = link ? *link : none;
  B200_REQUIRE(!lk.out16 || (out_kind == B200DEC_OUT_F32_ADD && ((uintptr_t)lk.out16 & 7) == 0 && lk.next_gamma &&
                             lk.stats_out && ((uintptr_t)lk.next_gamma & 15) == 0),
               "linear: the fp16 operand for the next LayerNorm goes with OUT_F32_ADD, its gamma and the sums");
  B200_REQUIRE(lnorm != 2 || (lk.stats_in && lk.stats_slots >= 1 && lk.stats_slots <= 128 && ((uintptr_t)lk.stats_in & 7) == 0),
               "linear: fp16 LayerNorm rows come with their partial sums (link->stats_in, stats_slots)");
  if (lnorm)
    B200_REQUIRE(ln->w && w->ln_g && w->ln_bias && w->k == D_MODEL,
                 "linear: the folded LayerNorm needs gamma, the weight's ln_g / ln_bias vectors and K = %d", D_MODEL);
  if (w->kind == B200DEC_W_INT8_24) B200_REQUIRE(w->meta, "linear: 2:4 weights need selectors");
  if (!head) {
    B200_REQUIRE(out && ((uintptr_t)out & 15) == 0 && ldo % 4 == 0 && ldo >= w->n, "linear: out / ldo");
    B200_REQUIRE(out_kind >= 0 && out_kind <= 2, "linear: out_kind");
  } else {
    B200_REQUIRE(pmax && pidx, "head: null partials");
  }
  // K = 4096 at more than 64 rows with fp32 or bf16 operands: the 128-row tile takes a whole SM's shared memory, and
  // clusters of eight such CTAs could not all be placed at once (some started 9 us late); two passes of 64 rows are
  // faster. fp16 rows on int8 / 2:4 weights are dealt over four CTAs of 32 rows per tile instead (one pass).
  const bool two_pass_wide = rows > 64 && w->k == 4096 && (split || lnorm != 0 || w->kind == B200DEC_W_BF16);
  if (rows > 64 && (two_pass_wide || !fits_any(w->kind, split, lnorm, w->warps, w->k, w->ksplit, rows)) &&
      fits_any(w->kind, split, lnorm, w->warps, w->k, w->ksplit, 64)) {
    // this operand does not fit shared memory for 128 rows at this K slice: two passes of up to 64 rows (the weights
    // are read twice; projections sized with b200dec_linear_fits avoid this)
    const size_t asz = (split || lnorm == 1) ? 4 : 2, osz = out_kind == B200DEC_OUT_F16 ? 2 : 4;
    const int np = head ? (w->n / (16 * w->warps)) * w->ksplit : 0;
    const int rc = run_linear(w, a, a_kind, ln, lda, 64, out, out_kind, ldo, act, pmax, pidx, logits, head, pdl, stream,
                              link, pf);
    if (rc) return rc;
    b200dec_ln_link up = lk;  // the second pass: the same link 64 rows further
    if (up.out16) up.out16 = (char*)up.out16 + (size_t)64 * ldo * 2;
    if (up.stats_out) up.stats_out += (size_t)64 * 2 * b200dec_linear_stat_slots(w);
    if (up.stats_in) up.stats_in += (size_t)64 * 2 * up.stats_slots;
    return run_linear(w, (const char*)a + (size_t)64 * lda * asz, a_kind, ln, lda, rows - 64,
                      out ? (char*)out + (size_t)64 * ldo * osz : nullptr, out_kind, ldo, act,
                      pmax ? pmax + (size_t)64 * np : nullptr, pidx ? pidx + (size_t)64 * np : nullptr,
                      logits ? logits + (size_t)64 * w->n : nullptr, head, pdl, stream, link ? &up : nullptr);
  }
  LinArgs p{};
  p.w = (const uint8_t*)w->w, p.meta = (const uint32_t*)w->meta, p.scale = w->scale, p.bias = w->bias;
  p.a = a, p.out = out, p.part_max = pmax, p.part_idx = pidx, p.logits = logits;
  p.next_gamma = lk.next_gamma, p.out16 = (__half*)lk.out16, p.stats_out = lk.stats_out;
  p.stats_in = lk.stats_in, p.stats_slots = lk.stats_slots;
  if (lnorm) p.ln_w = ln->w, p.ln_g = w->ln_g, p.ln_bias = w->ln_bias, p.ln_eps = ln->eps;
  p.lda = lda, p.ldo = ldo, p.rows = rows, p.N = w->n, p.out_kind = out_kind, p.act = act, p.head = head;
  if (pf) p.pf = *pf;
  p.status = lk.status;
  cudaStream_t s = (cudaStream_t)stream;
  switch (w->kind) {
    case B200DEC_W_INT8: return launch_int8(p, split, lnorm, w->warps, w->k, w->ksplit, pdl, s);
    case B200DEC_W_INT8_24: return launch_24(p, split, lnorm, w->warps, w->k, w->ksplit, pdl, s);
    case B200DEC_W_BF16: return launch_bf16(p, split, lnorm, w->warps, w->k, w->ksplit, pdl, s);
    case B200DEC_W_F16: return launch_f16(p, split, lnorm, w->warps, w->k, w->ksplit, pdl, s);
  }
  return fail(B200DEC_EINVAL, "linear: weight kind %d", w->kind);
}

}  // namespace

namespace b200dec_detail {
// launches one call of linear_impl makes (1, or 2 when the rows go in two passes)
int linear_passes(const b200dec_weight* w, int a_kind, bool ln, int rows) {
  if (is_umma_kind(w->kind)) return 1;  // more than 64 rows of K = 4096 are dealt over grid.z of one launch
  const bool split = a_kind == B200DEC_A_F32_SPLIT;
  const int lnorm = !ln ? 0 : a_kind == B200DEC_A_F16_ROWS16 ? 2 : 1;
  const bool two_pass_wide = rows > 64 && w->k == 4096 && (split || lnorm != 0 || w->kind == B200DEC_W_BF16);
  return (rows > 64 && (two_pass_wide || !fits_any(w->kind, split, lnorm, w->warps, w->k, w->ksplit, rows)) &&
          fits_any(w->kind, split, lnorm, w->warps, w->k, w->ksplit, 64)) ? 2 : 1;
}
int linear_impl(const b200dec_weight* w, const void* a, int a_kind, const b200dec_norm* ln, int lda, int rows, void* out,
                int out_kind, int ldo, int act, int pdl, void* stream, const b200dec_ln_link* link,
                const KvPrefetch* pf) {
  return run_linear(w, a, a_kind, ln, lda, rows, out, out_kind, ldo, act, nullptr, nullptr, nullptr, 0, pdl, stream,
                    link, pf);
}
int head_impl(const b200dec_weight* w, const void* a, int a_kind, const b200dec_norm* ln, int lda, int rows, float* pmax,
              int* pidx, float* logits, int pdl, void* stream) {
  return run_linear(w, a, a_kind, ln, lda, rows, nullptr, B200DEC_OUT_F32, 0, B200DEC_ACT_NONE, pmax, pidx, logits, 1,
                    pdl, stream);
}
}  // namespace b200dec_detail

extern "C" {

int b200dec_linear(const b200dec_weight* w, const void* a, int a_kind, const b200dec_norm* ln, int lda, int rows,
                   void* out, int out_kind, int ldo, int act, int pdl, void* stream) {
  return linear_impl(w, a, a_kind, ln, lda, rows, out, out_kind, ldo, act, pdl, stream, nullptr, nullptr);
}

int b200dec_linear_linked(const b200dec_weight* w, const void* a, int a_kind, const b200dec_norm* ln, int lda, int rows,
                          void* out, int out_kind, int ldo, int act, const b200dec_ln_link* link, int pdl,
                          void* stream) {
  return linear_impl(w, a, a_kind, ln, lda, rows, out, out_kind, ldo, act, pdl, stream, link, nullptr);
}

int b200dec_head_argmax(const b200dec_weight* w, const void* a, int a_kind, const b200dec_norm* ln, int lda, int rows,
                        float* part_max, int32_t* part_idx, float* logits, int pdl, void* stream) {
  return head_impl(w, a, a_kind, ln, lda, rows, part_max, part_idx, logits, pdl, stream);
}

int b200dec_linear_stat_slots(const b200dec_weight* w) {
  if (!w) return 0;
  return is_umma_kind(w->kind) ? (w->n / 128) * w->ksplit : (w->n / (16 * w->warps)) * w->ksplit;
}

int b200dec_head_partials(const b200dec_weight* w) {
  if (!w) return 0;
  return is_umma_kind(w->kind) ? w->n / 128 : (w->n / (16 * w->warps)) * w->ksplit;
}

int b200dec_linear_fits(int kind, int a_kind, int ln, int warps, int ksplit, int k, int rows) {
  if (ksplit < 1 || k % ksplit) return 0;
  const int mode = ln == 0 ? 0 : a_kind == B200DEC_A_F16_ROWS16 ? 2 : 1;
  return fits_any(kind, a_kind == B200DEC_A_F32_SPLIT, mode, warps, k, ksplit, rows) ? 1 : 0;
}

int64_t b200dec_tiled_bytes(int kind, int n, int k) {
  if (kind == B200DEC_W_INT8 || kind == B200DEC_W_INT8_UMMA) return (int64_t)n * k;
  if (kind == B200DEC_W_BF16 || kind == B200DEC_W_F16 || kind == B200DEC_W_F16_UMMA) return (int64_t)n * k * 2;
  if (kind == B200DEC_W_INT8_24 || kind == B200DEC_W_INT8_24_UMMA) return (int64_t)n * k / 2;
  return -1;
}
int64_t b200dec_tiled_meta_bytes(int kind, int n, int k) {
  return kind == B200DEC_W_INT8_24 || kind == B200DEC_W_INT8_24_UMMA ? (int64_t)n * k / 8 : 0;
}

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
