/* b200dec: C-ABI of the B200 (sm_100a) decoder token loop.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as void*, a cudaStream_t), launches
 * on that stream and returns 0, or a nonzero code with a message in b200dec_last_error(). No entry point allocates,
 * frees, synchronises or throws, so all of them may be called while the stream is being captured into a CUDA graph.
 * The caller owns every buffer. Citations name the interface of the reference project (kadirnar/cohere-inference) that
 * each entry point replaces, as file:line inside that project.
 *
 * Conventions: d_model is 1024; "rows" are the rows of one decoding step (row r works on slot active[r]); a16 = IEEE
 * half activations, f32 = float. Weight matrices are (N, K) row-major on the reference side and are re-tiled once by
 * the b200dec_tile_* calls into the streaming layout of the GEMM kernels (described in csrc/linear.cu).
 */
#ifndef B200DEC_H
#define B200DEC_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { B200DEC_W_BF16 = 0, B200DEC_W_INT8 = 1, B200DEC_W_INT8_24 = 2,     /* weight storage of one projection */
       B200DEC_W_INT8_UMMA = 3,    /* int8 in the block layout of the tcgen05 kernels (b200dec_tile_int8_umma): the
                                      vocabulary projection (b200dec_head_umma) and, through b200dec_linear_linked,
                                      layer projections on fp16 rows (a_kind B200DEC_A_F16, or B200DEC_A_F16_ROWS16
                                      with a LayerNorm): N a multiple of 128, K = 1024 with w->ksplit 4 or 8, or
                                      K = 4096 with w->ksplit 8 and no LayerNorm */
       B200DEC_W_F16 = 4,          /* fp16 values in the layout of B200DEC_W_BF16 (b200dec_tile_bf16 moves 16-bit
                                      words): no scale; multiplied as fp16 x fp16 with fp32 accumulation, so it takes
                                      every operand kind and tile the int8 weights take (fp16 rows, the linked
                                      LayerNorm, rows dealt over CTAs) */
       B200DEC_W_F16_UMMA = 5,     /* fp16 values as the images of the tcgen05 kernels' swizzled shared-memory tiles
                                      (b200dec_tile_f16_umma), copied there from HBM by cp.async.bulk: no scale; the
                                      shapes and calls of B200DEC_W_INT8_UMMA, the vocabulary projection only through
                                      b200dec_head_umma_linked */
       B200DEC_W_INT8_24_UMMA = 6 }; /* 2:4 int8 (kept values + selector words, b200dec_tile_24_umma) for the tcgen05
                                      projection kernel, which expands them to dense tiles: the layer-projection
                                      shapes and calls of B200DEC_W_INT8_UMMA (not the vocabulary projection) */
enum { B200DEC_A_F16 = 0, B200DEC_A_F32_SPLIT = 1,  /* activation operand of a projection: one fp16, or hi + lo */
       B200DEC_A_F16_ROWS16 = 2 };  /* one fp16, and with a LayerNorm the rows handed in are its ready fp16 operand
                                      (see b200dec_ln_link) */
enum { B200DEC_OUT_F16 = 0, B200DEC_OUT_F32 = 1, B200DEC_OUT_F32_ADD = 2 };/* store, or add into an fp32 residual */
enum { B200DEC_ACT_NONE = 0, B200DEC_ACT_RELU = 1, B200DEC_ACT_GELU = 2 };
enum { B200DEC_OK = 0, B200DEC_EINVAL = 1, B200DEC_ECUDA = 2, B200DEC_EARCH = 3 };

/* bits of the device status word (written by kernels, never cleared by them) */
enum { B200DEC_ST_TOKEN_RANGE = 1, B200DEC_ST_POS_RANGE = 2, B200DEC_ST_FRAMES_RANGE = 4, B200DEC_ST_SLOT_RANGE = 8,
       B200DEC_ST_TIMEOUT = 16 /* a bounded wait inside a kernel ran out; the kernel returned without its result */ };

/* One projection y = a W^T (* scale) + bias in the tiled layout. */
typedef struct b200dec_weight {
  const void* w;       /* tiled weights: int8 (+128), bf16, or the kept values of a 2:4 matrix */
  const void* meta;    /* tiled 2:4 selectors, else NULL */
  const float* scale;  /* per output channel, int8 kinds; NULL for bf16 */
  const float* bias;   /* per output channel or NULL */
  const float* ln_g;   /* for a projection called with a folded LayerNorm: g[n] = sum_k gamma[k] W[n][k] ... */
  const float* ln_bias;/* ... and sum_k beta[k] W[n][k], of the dequantised weights W; else NULL */
  int32_t n, k;        /* logical shape */
  int32_t kind;        /* B200DEC_W_* */
  int32_t warps;       /* output tile of a CTA = 16 * warps channels (4 or 8) */
  int32_t ksplit;      /* CTAs of a cluster sharing K (1, 2, 4 or 8): K / ksplit in {128, 256, 512} */
} b200dec_weight;

typedef struct b200dec_norm {
  const float* w;
  const float* b;
  float eps;
  int32_t _pad;
} b200dec_norm;

typedef struct b200dec_layer {
  b200dec_norm ln1, ln2, ln3;
  b200dec_weight qkv, o, cq, co, fc1, fc2;
  void* self_k;   /* bf16, or int8 when the plan's kv_int8 is set, (slots + 1, H, seq, D) */
  void* self_v;
  const void* cross_k; /* bf16 or int8 (slots + 1, H, frames, D) */
  const void* cross_v;
  float* self_ks;      /* kv_int8: one fp32 scale per cached vector, (slots + 1, H, seq); else NULL */
  float* self_vs;
  float* cross_ks;     /* (slots + 1, H, frames) */
  float* cross_vs;
} b200dec_layer;

/* Everything one decoding step touches. Replaces the argument lists of StreamDecoder._step
 * (kernels/stream_decoder.py:176-199). */
typedef struct b200dec_plan {
  int32_t layers, heads, head_dim, act;      /* act: B200DEC_ACT_* of the feed-forward */
  int32_t slots, seq, frames, vocab;         /* dummy slot = slots; caches hold seq / frames positions */
  int32_t max_prompt, out_cols, pad, eos;    /* forced (slots+1, max_prompt), out (slots+1, out_cols) */
  int32_t a_kind, max_pos;                   /* B200DEC_A_*: operand precision of the layer projections */
  int32_t head_a_kind, pdl;                  /* operand precision of the vocabulary projection; pdl: which launches are
                                                programmatic (1 projection after projection, 2 attention, 4 projection
                                                after attention) */
  int32_t attn_ring, kv_int8;                /* attn_ring != 0: the attention kernels are b200dec_attention_ring;
                                                kv_int8 != 0: int8 caches with per-vector scales (the layers'
                                                self_ks .. cross_vs), attention by the *_q8 entry points */
  int32_t kv_prefetch_mb;                    /* > 0 (and a step of rows * heads >= 512 with both schedules): the output
                                                projection after self-attention starts the layer's cross keys and
                                                values on their way into L2, the one after cross-attention the next
                                                layer's self keys and values, up to this many MB per attention launch
                                                (the projections leave HBM idle; L2 holds 126 MB); 0: off */
  int32_t wait_limit, withhold;              /* as in b200dec_ln_link, for the step's tcgen05 kernels; withhold bit 0
                                                the vocabulary projection, bit 1 the layer projections (tests only) */
  int32_t classes;                           /* 0: the whole step. Else only these kernels are launched (a timing aid:
                                                the results are then meaningless): 1 embedding + vocabulary projection
                                                + pick, 2 the layer projections, 4 the attention kernels */
  const void* embed;  /* bf16 (vocab, 1024) */
  const void* pos_table; /* bf16 (max_pos, 1024) */
  b200dec_norm emb_ln, final_ln;
  const b200dec_layer* layer;  /* host array of `layers` entries */
  b200dec_weight head;
  /* slot state (slots + 1 entries each) */
  const int32_t* active;  /* (rows) */
  int64_t* tok;
  int32_t* pos;
  const int32_t* plen;
  const int32_t* limit;
  const int32_t* cross_len;
  uint8_t* finished;
  const int64_t* forced;
  int64_t* out;
  uint8_t* flags_host;    /* NULL, or (slots + 1) bytes of pinned host memory as the device addresses it: a row that
                             ends at a step sets its slot's byte there (the pick kernel, one posted write), so the host
                             reads the flags after the step's event without a device-to-host copy in the step (the
                             reference's step ends with that copy, kernels/stream_decoder.py:199); the host clears a
                             slot's byte when it admits into it (kernels/stream_decoder.py:263) */
  int32_t* status;        /* one word, B200DEC_ST_* bits */
  /* scratch owned by the caller */
  float* x;       /* (max rows, 1024) residual stream */
  float* qkv;     /* (max rows, 3072) */
  float* cq;      /* (max rows, 1024) */
  void* att;      /* (max rows, 1024) a16 or f32 */
  void* mid;      /* (max rows, ffn) a16 or f32 */
  float* attn_part;    /* b200dec_attention_scratch_floats() floats */
  int32_t* attn_count; /* rows * heads counters, zero on entry and on exit */
  float* head_max;     /* (max rows, b200dec_head_partials()) */
  int32_t* head_idx;
  void* xh;             /* (max rows, 1024) fp16: the residual stream times the next LayerNorm's gamma, the operand of
                           the LayerNorm-folding projections (a_kind F16 only); NULL: they convert the fp32 rows */
  float* ln_stats;      /* (max rows, 128, 2) partial row sums that go with xh (see b200dec_ln_link) */
  int32_t* sched_self;  /* (max rows, 4) row schedules for b200dec_attention_paired, 16-byte aligned; both NULL: */
  int32_t* sched_cross; /* the step uses b200dec_attention for every batch size */
  /* optional recording (tests, teacher forcing); NULL in production */
  float* logits;       /* (rows, vocab) */
  int64_t* argmax;     /* (slots + 1): the un-forced greedy choice of each slot's last step */
} b200dec_plan;

const char* b200dec_last_error(void);
int b200dec_version(void);
/* sizeof the structures above as this library was compiled (which: 0 b200dec_weight, 1 b200dec_norm, 2 b200dec_layer,
 * 3 b200dec_plan, 4 b200dec_ln_link), so that a binding in another language can check its own layout. */
int b200dec_sizeof(int which);

/* ---- packing (init time) ------------------------------------------------------------------------------------ */

/* Per-row symmetric int8: s = max(absmax, 1e-12) / 127, q = clamp(rint(w / s), -127, 127).
 * Replaces quantize_rows (kernels/fast_encoder.py:60-63) and the arithmetic of prepare_w8
 * (kernels/stream_decoder.py:45-46). */
int b200dec_quantize_rows(const float* w, int n, int k, int8_t* q, float* scale, void* stream);
/* The reference's dec_w8_linear layout: uint8 = q + 128, bytes of every 16 along K permuted by W8_PERM.
 * Replaces prepare_w8 (kernels/stream_decoder.py:38-48), bit for bit. */
int b200dec_prepare_w8(const float* w, int n, int k, uint8_t* u8, float* scale, void* stream);
/* Zero the two smallest |w| of every four along K (lower index first on ties).
 * Replaces prune_24_magnitude (kernels/sparse.py:42-46). */
int b200dec_prune24(const float* w, int n, int k, float* out, void* stream);
/* kept values (n, k/2) and selector words (n, k/32) of a 2:4 int8 matrix; *bad (device) is set to 1 if some group
 * of four holds more than two nonzeros. Replaces compress_24 (kernels/sparse.py:26-39), bit for bit. */
int b200dec_compress24(const int8_t* q, int n, int k, int8_t* kept, int32_t* words, int32_t* bad, void* stream);
/* Streaming layouts of the GEMM kernels (no counterpart in the reference: its layout is prepare_w8's). */
int64_t b200dec_tiled_bytes(int kind, int n, int k);      /* bytes of the weight part */
int64_t b200dec_tiled_meta_bytes(int kind, int n, int k); /* bytes of the selector part (0 unless 2:4) */
int b200dec_tile_int8(const int8_t* q, int n, int k, void* tiled, void* stream);
int b200dec_tile_bf16(const void* w_bf16, int n, int k, void* tiled, void* stream);
int b200dec_tile_f16_umma(const void* w_f16, int n, int k, void* tiled, void* stream); /* n % 128 == 0, k % 64 == 0 */
int b200dec_tile_24(const int8_t* kept, const int32_t* words, int n, int k, void* tiled, void* meta, void* stream);
int b200dec_tile_24_umma(const int8_t* kept, const int32_t* words, int n, int k, void* tiled, void* meta,
                         void* stream); /* n % 128 == 0, k % 64 == 0 */

/* ---- step kernels ------------------------------------------------------------------------------------------- */

/* x = LN_emb(embed[tok[s]] + pos_table[pos[s]]) and, when hn is not NULL, hn = LN_1(x); s = active[r] in 0..slots
 * (slots = the dummy).
 * Replaces dec_embed (kernels/csrc/decoder_ops.cu:24-54, 208-219). */
int b200dec_embed_ln(const int32_t* active, const int64_t* tok, const int32_t* pos, const void* embed,
                     const void* pos_table, int vocab, int max_pos, int slots, b200dec_norm ln0, b200dec_norm ln1,
                     float* x, void* hn, int hn_kind, int rows, int32_t* status, int pdl, void* stream);
/* hn = LN(x) for an fp32 residual stream that the preceding projection already added into
 * (B200DEC_OUT_F32_ADD). Replaces dec_add_ln (kernels/csrc/decoder_ops.cu:56-83, 221-231). The step itself does not
 * launch it: its projections normalise while staging their operand (the `ln` argument of b200dec_linear). */
int b200dec_layer_norm(const float* x, b200dec_norm ln, void* hn, int hn_kind, int rows, int pdl, void* stream);
/* out = act(a' W^T * scale + bias) for rows <= 128, where a' = a, or LayerNorm(a) of the fp32 rows a when ln is not
 * NULL (then K = 1024, a_kind only selects the operand precision, and w->ln_g / w->ln_bias must have been computed
 * from ln's gamma and beta). Replaces dec_w8_linear
 * (kernels/csrc/dec_w8.cu:46-234), the Triton _linear (kernels/decoder_kernels.py:19-66), the cuBLAS F.linear of
 * kernels/stream_decoder.py:23-27 and, with ln, the dec_add_ln in front of it (kernels/csrc/decoder_ops.cu:56-83). */
int b200dec_linear(const b200dec_weight* w, const void* a, int a_kind, const b200dec_norm* ln, int lda, int rows,
                   void* out, int out_kind, int ldo, int act, int pdl, void* stream);
/* Links between a projection that updates the residual stream (B200DEC_OUT_F32_ADD) and the LayerNorm-folding
 * projection that reads it next, so that the reader stages a ready fp16 operand with asynchronous copies instead of
 * converting fp32 rows. The producer (next_gamma, out16, stats_out set) also writes out16 (rows, ldo) = updated row *
 * next_gamma as fp16 and, per row, one partial (sum, sum of squares) for each of its b200dec_linear_stat_slots(w)
 * finishing CTAs: stats_out (rows, slots, 2) fp32. The reader (ln != NULL, a_kind = B200DEC_A_F16_ROWS16, a = that
 * out16, int8 or 2:4 weights with a K slice <= 256) adds up stats_in (rows, stats_slots, 2) in a fixed order.
 * b200dec_ln_rows16 starts a chain from fp32 rows: out16 = x * gamma and one slot of sums per row. Same reference
 * counterparts as b200dec_linear and b200dec_layer_norm. */
typedef struct b200dec_ln_link {
  const float* next_gamma;
  void* out16;
  float* stats_out;
  const float* stats_in;
  int32_t stats_slots;
  int32_t wait_limit; /* B200DEC_W_INT8_UMMA: polls before the wait for the MMAs gives up; 0 = the default (2^22) */
  int32_t* status;  /* required with a B200DEC_W_INT8_UMMA weight (reader, producer or neither): the status word
                       that receives B200DEC_ST_TIMEOUT if the bounded wait for the MMAs ran out; the mma.sync kinds
                       report there if the bounded wait for their cluster's partial results ran out (tiles that
                       exchange them by st.async) */
  int32_t withhold; /* tests only, B200DEC_W_INT8_UMMA: nonzero leaves out the MMAs' completion signal, so the wait
                       runs out, the status word gets B200DEC_ST_TIMEOUT and the kernel returns; 0 in production */
} b200dec_ln_link;
int b200dec_linear_linked(const b200dec_weight* w, const void* a, int a_kind, const b200dec_norm* ln, int lda, int rows,
                          void* out, int out_kind, int ldo, int act, const b200dec_ln_link* link, int pdl,
                          void* stream);
int b200dec_linear_stat_slots(const b200dec_weight* w);
int b200dec_ln_rows16(const float* x, const float* gamma, int rows, void* out16, float* stats, void* stream);
/* 1 when a projection with this tile (warps, ksplit) fits shared memory for `rows` rows in one pass (else the call
 * makes two passes of up to 64 rows and reads the weights twice). Host-only query. */
int b200dec_linear_fits(int kind, int a_kind, int ln, int warps, int ksplit, int k, int rows);
/* Vocabulary projection fused with the per-tile argmax: writes, per row, b200dec_head_partials(w) (max, first index)
 * pairs; logits (rows, n) fp32 optional. Replaces the head projection + the scan of dec_pick
 * (kernels/stream_decoder.py:173-174, 197; kernels/csrc/decoder_ops.cu:106-147). */
int b200dec_head_argmax(const b200dec_weight* w, const void* a, int a_kind, const b200dec_norm* ln, int lda, int rows,
                        float* part_max, int32_t* part_idx, float* logits, int pdl, void* stream);
int b200dec_head_partials(const b200dec_weight* w);
/* The same vocabulary projection on the fifth-generation tensor cores (tcgen05.mma, accumulator in tensor memory):
 * x (rows, lda) fp32 is normalised by ln inside the kernel (ln is required), w->kind must be B200DEC_W_INT8_UMMA
 * (w->w from b200dec_tile_int8_umma, K = 1024, N a multiple of 128; w->warps, ksplit, ln_g, ln_bias unused) and the
 * partials are one per 128 channels (b200dec_head_partials() = N / 128). rows <= 128 (above 64 rows a second set of
 * CTAs of the same launch takes rows 64..; the weights come from HBM once). Replaces the same
 * reference code as b200dec_head_argmax. status receives B200DEC_ST_TIMEOUT if a bounded wait ran out. */
int b200dec_head_umma(const b200dec_weight* w, const float* x, const b200dec_norm* ln, int lda, int rows,
                      float* part_max, int32_t* part_idx, float* logits, int32_t* status, int pdl, void* stream);
/* The same with the LayerNorm's input handed over as in b200dec_ln_link: xg (rows, lda) fp16 = row * gamma (the out16
 * of the projection that produced the rows, or of b200dec_ln_rows16) and its partial sums stats (rows, stats_slots,
 * 2); the normalisation is folded into the epilogue with w->ln_g / w->ln_bias (ln supplies eps). */
int b200dec_head_umma_linked(const b200dec_weight* w, const void* xg, const float* stats, int stats_slots,
                             const b200dec_norm* ln, int lda, int rows, float* part_max, int32_t* part_idx,
                             float* logits, int32_t* status, int pdl, void* stream);
/* q (n, k) int8 row-major (b200dec_quantize_rows) -> the 8 KB block layout of b200dec_head_umma, n*k bytes. */
int b200dec_tile_int8_umma(const int8_t* q, int n, int k, void* tiled, void* stream);
/* Greedy choice from the partials, prompt forcing, output row, position advance, end flag; rows on the dummy slot and
 * finished slots change nothing. flags_host: NULL, or pinned host memory (device-addressable) in which a row that ends
 * at this step sets its slot's byte. Replaces the bookkeeping of dec_pick (kernels/csrc/decoder_ops.cu:148-159, 304-314). */
int b200dec_pick(const float* part_max, const int32_t* part_idx, int partials, const int32_t* active, int rows,
                 int dummy, int64_t* tok, int32_t* pos, uint8_t* finished, const int64_t* forced, int max_prompt,
                 const int32_t* plen, const int32_t* limit, int64_t* out, int out_cols, int eos, int64_t* argmax,
                 uint8_t* flags_host, int pdl, void* stream);
/* One new token per row against its slot's cache. self != 0: q | k | v in qkv (rows, 3 * H * D) fp32, the new key and
 * value are written at n[s] and attended, keys 0..n[s]; else q (rows, H * D) over n[s] frames. Caches bf16
 * (slots + 1, H, cap, D). Replaces dec_attention (kernels/csrc/decoder_ops.cu:85-104, 235-261; dec_attn.cuh:84-188). */
int b200dec_attention(int self, const int32_t* active, const float* q, int ldq, void* kcache, void* vcache,
                      const int32_t* n, int slots, int heads, int head_dim, int cap, float scale, void* out,
                      int out_kind, int rows, float* part, int32_t* count, int32_t* status, int pdl, void* stream);
int64_t b200dec_attention_scratch_floats(int rows, int heads, int head_dim);
/* b200dec_attention over int8 caches (slots + 1, H, cap, D) with one fp32 scale per cached key vector and value
 * vector (slots + 1, H, cap): x ~ q * scale, scale = absmax / 127 (1 for a zero vector), q = rint(clamp(x / scale)).
 * self != 0 rounds the row's new key and value to bf16, writes their int8 form and scales at n[s], and attends them
 * in this step as the bf16 values. Replaces dec_attention_q8 (kernels/csrc/decoder_ops.cu:263-290;
 * dec_attn.cuh:38-63, 100-106, 116-152). */
int b200dec_attention_q8(int self, const int32_t* active, const float* q, int ldq, void* kcache, void* vcache,
                         float* kscale, float* vscale, const int32_t* n, int slots, int heads, int head_dim, int cap,
                         float scale, void* out, int out_kind, int rows, float* part, int32_t* count, int32_t* status,
                         int pdl, void* stream);
/* The step's rows ranked by decreasing length, for b200dec_attention_paired: sched_self from pos[slot] (keys in the
 * self cache), sched_cross from cross_len[slot] (encoder frames); either table may be NULL. Entry i of a table is
 * int32 {row, slot, length, prefetch} of the row of rank i (ties by row), lengths clamped into 0..seq-1 / 1..frames and
 * slots into 0..slots with the status bits of b200dec_attention. prefetch = how many of the row's keys the projections
 * before the attention launch bring into L2 ahead of it (see b200dec_plan.kv_prefetch_mb): all of them when the
 * table's lengths add up to at most prefetch_keys, else in proportion; 0 with prefetch_keys = 0. rows <= 256.
 * b200dec_step builds both tables with an extra CTA of its embedding kernel; this entry point is for hosts that launch
 * the kernels themselves. No counterpart in the reference (its attention takes rows in batch order,
 * kernels/csrc/dec_attn.cuh:84-188). */
int b200dec_row_schedule(const int32_t* active, const int32_t* pos, const int32_t* cross_len, int slots, int seq,
                         int frames, int rows, int prefetch_keys, int32_t* sched_self, int32_t* sched_cross,
                         int32_t* status, void* stream);
/* b200dec_attention for a large batch (rows * heads >= 512 is where it pays), reading the rows from a schedule: the
 * i-th longest row and the i-th shortest share a cluster of two CTAs that read the same number of keys; the partial
 * of the long row's tail crosses distributed shared memory. Same results as b200dec_attention up to the order of the
 * softmax merge. sched: (rows, 4) int32 from b200dec_row_schedule, 16-byte aligned. With pdl != 0 the kernel reads its
 * schedule entries before it waits for its predecessor on the stream: the schedule must then be complete before that
 * predecessor starts, i.e. at least one kernel must lie between the one that writes the schedule and this launch
 * (the two CTAs of a pair must see the same entries); launch with pdl = 0 directly behind the schedule's writer. */
int b200dec_attention_paired(int self, const int32_t* sched, const float* q, int ldq, void* kcache, void* vcache,
                             int heads, int head_dim, int cap, float scale, void* out, int out_kind, int rows,
                             int pdl, void* stream);
/* The same over int8 caches (see b200dec_attention_q8). */
int b200dec_attention_paired_q8(int self, const int32_t* sched, const float* q, int ldq, void* kcache, void* vcache,
                                float* kscale, float* vscale, int heads, int head_dim, int cap, float scale, void* out,
                                int out_kind, int rows, int pdl, void* stream);
/* The same operation, arguments and workspace as b200dec_attention (rows <= 128) by a persistent kernel: two CTAs
 * per SM, one producer lane streaming (row, head) caches through a shared-memory ring with cp.async.bulk and
 * mbarriers, four consumer warps. Smaller footprint per SM; see csrc/attention_ring.cu. */
int b200dec_attention_ring(int self, const int32_t* active, const float* q, int ldq, void* kcache, void* vcache,
                           const int32_t* n, int slots, int heads, int head_dim, int cap, float scale, void* out,
                           int out_kind, int rows, float* part, int32_t* count, int32_t* status, int pdl, void* stream);
/* b200dec_attention for a caller that cannot provide the split workspace because it must not allocate device memory
 * where it calls this (a frozen memory pool, a plugin ABI that passes only inputs and outputs, a foreign runtime that
 * would not see the allocation). No counterpart in the reference. The workspace is an array inside the library
 * instead (4.3 MB per GPU, held until the process exits), good for rows * heads <= 512; larger calls are refused
 * with an error. The first call on each device looks the array's address up and should come before any stream
 * capture. The device that is current at the call must be the device of `stream`: the array's address is looked up
 * for the current device. All calls on a device share the array: two calls whose kernels overlap on the GPU
 * (different streams) race on it. `pdl` is accepted and not used: the call first clears its arrival counters with a
 * memset on `stream`, so the kernel's predecessor is never a kernel. After the first call it may be captured into a
 * CUDA graph (memset node + kernel node) and replayed. Allocates nothing, frees nothing. */
int b200dec_attention_static(int self, const int32_t* active, const float* q, int ldq, void* kcache, void* vcache,
                             const int32_t* n, int slots, int heads, int head_dim, int cap, float scale, void* out,
                             int out_kind, int rows, int32_t* status, int pdl, void* stream);
/* Packed cross keys/values kv (nrows, L * 2 * H * D) fp32, row i = frame frame_of[i] of slot slot_of[i], into the
 * bf16 slot caches (L, slots + 1, H, frames, D). Replaces dec_scatter_kv (kernels/csrc/decoder_ops.cu:163-173,
 * 316-327). */
int b200dec_scatter_kv(const float* kv, const int32_t* slot_of, const int32_t* frame_of, void* ck, void* cv,
                       int nrows, int layers, int slots_plus_1, int heads, int head_dim, int frames, void* stream);
/* The same into int8 caches with fp32 scales (L, slots + 1, H, frames): every head vector is rounded to bf16, then
 * quantised as in b200dec_attention_q8. Replaces dec_scatter_kv_q8 (kernels/csrc/decoder_ops.cu:175-204). */
int b200dec_scatter_kv_q8(const float* kv, const int32_t* slot_of, const int32_t* frame_of, void* ck, void* cv,
                          float* ck_scale, float* cv_scale, int nrows, int layers, int slots_plus_1, int heads,
                          int head_dim, int frames, void* stream);
/* A measurement aid, no counterpart in the reference and not a step of the decoder: `ctas` CTAs of 128 threads each
 * read `bytes_per_cta` contiguous bytes of src (CTA c from src + c * bytes_per_cta) with the attention kernels' loads
 * (16 bytes per thread, streaming, 8 in flight) and do nothing else. The time of such a launch is what a kernel of
 * that grid and that many bytes can read at all, ramp-up and tail included; bench.py reports the attention kernel
 * against it. src: 16-byte aligned, at least ctas * bytes_per_cta bytes; sink: NULL or one word (never written in
 * practice). */
int b200dec_read_probe(const void* src, int ctas, int64_t bytes_per_cta, int32_t* sink, int pdl, void* stream);
/* ---- cross-attention prefill (fill_cross) on the tcgen05 tensor cores ----------------------------------------------
 * C(m, n) = A(m, k) W(n, k)^T + bias with fp32 rows A (used as two bf16 halves, about 16 bits of mantissa), bf16
 * weights and fp32 accumulation; the result goes (mode 0) into the operand image of the next product, or (modes 1, 2)
 * straight into the slot caches. Together these replace the two chained F.linear of StreamDecoder.fill_cross
 * (kernels/stream_decoder.py:229-239) and dec_scatter_kv / dec_scatter_kv_q8 (kernels/csrc/decoder_ops.cu:163-204,
 * 292-327): no (frames x layers * 2 * d) intermediate exists and the host builds no per-frame index vectors.
 * Operands live in global memory as images of their shared-memory tiles: */
int64_t b200dec_prefill_rows_bytes(int m, int k); /* bytes of the image of m fp32 rows of k values (k % 64 == 0) */
/* x (m, ldx) fp32 -> its image (1 KB aligned, b200dec_prefill_rows_bytes(m, k) bytes). */
int b200dec_prefill_pack_rows(const float* x, int m, int k, int ldx, void* image, void* stream);
/* w (n, k) bf16 row-major (n % 256 == 0, k % 64 == 0) -> its image (1 KB aligned, n * k * 2 bytes); init time. */
int b200dec_prefill_tile_weight(const void* w_bf16, int n, int k, void* image, void* stream);
/* mode 0: next_image = the image of the m result rows (n values each) for the next product.
 * mode 1: n = layers * 2 * heads * head_dim; row r of the product is frame (r - first) of the slot of the piece that
 *   holds it, pieces (n_pieces, 4) int32 {first row, frames, slot, 0} in device memory, first rows ascending from 0;
 *   channel ((layer * 2 + kv) * heads + head) * head_dim + d goes to the bf16 cache (layers, slots_plus_1, heads,
 *   frames, head_dim) of keys (kv = 0) or values. Rows outside every piece or past the cache are dropped.
 * mode 2: the same into int8 caches with one fp32 scale per head vector (layers, slots_plus_1, heads, frames),
 *   quantised as b200dec_scatter_kv_q8 does.
 * status receives B200DEC_ST_TIMEOUT if a bounded wait inside the kernel ran out. */
int b200dec_prefill_gemm(const void* rows_image, int m, int k, const void* weight_image, const float* bias, int n,
                         int mode, void* next_image, const int32_t* pieces, int n_pieces, void* ck, void* cv,
                         float* ck_scale, float* cv_scale, int layers, int slots_plus_1, int heads, int head_dim,
                         int frames, int32_t* status, void* stream);
/* Admission of n requests in one launch. records: n packed records of b200dec_admit_record_ints(max_prompt) int32 in
 * device memory (the host stages them in pinned memory and copies them over in one piece): {slot, prompt length,
 * new-token budget, encoder frames, max_prompt token ids}. Per record: forced = the prompt padded with `pad`, out =
 * the prompt then `pad`, tok = prompt[0], pos = 0, plen, limit = plen - 1 + budget, cross_len = frames, finished = 0.
 * A slot outside 0..slots-1 is skipped, a prompt length or frame count out of range is clamped, both with a status bit.
 * n_active != NULL: the slots are also appended, in record order, to plan->active at position *n_active (a device
 * word, advanced by the kernel; max_rows = the list's capacity). Replaces StreamDecoder.admit
 * (kernels/stream_decoder.py:241-263): one copy and one kernel instead of nine indexed writes and seven copies. */
int b200dec_admit(const b200dec_plan* plan, const int32_t* records, int n, int32_t* n_active, int max_rows,
                  void* stream);
int b200dec_admit_record_ints(int max_prompt);
/* Tail of a step when the active list lives on the device: the rows of plan->active[0 .. rows) whose slot has not
 * ended move to the front in their order, the rest point at the dummy slot, *n_active = the live count (also written to
 * live_host, pinned host memory as the device addresses it, when not NULL). rows <= 128.
 * With it a host never rebuilds the list on eviction (it reads the end flags and the count the step leaves in pinned
 * memory); the flag scan and compaction of the reference's decoder thread (kernels/pipeline.py:217-231) on the GPU. */
int b200dec_compact_active(const b200dec_plan* plan, int rows, int32_t* n_active, int32_t* live_host, int pdl,
                           void* stream);
/* The whole step for `rows` rows: embed, `layers` layers, head, pick. Replaces StreamDecoder._step
 * (kernels/stream_decoder.py:176-199); its D2H copy of the flags becomes plan->flags_host, or stays with the caller. */
int b200dec_step(const b200dec_plan* plan, int rows, void* stream);
/* The same for rows [row0, row0 + rows) of the step's batch only. Disjoint row ranges share no scratch, so a caller
 * may run several ranges concurrently on forked streams to overlap one range's attention (bound by HBM) with another's
 * projections (bound by latency). No counterpart in the reference, which runs the batch as one chain. */
int b200dec_step_rows(const b200dec_plan* plan, int row0, int rows, void* stream);
/* Kernels b200dec_step launches for `rows` rows (for launch accounting). */
int b200dec_step_launches(const b200dec_plan* plan, int rows);

#ifdef __cplusplus
}
#endif
#endif
