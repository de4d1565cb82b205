// One decoding step as a sequence of kernel launches on the caller's stream (capturable into a CUDA graph):
// embed + embedding LayerNorm, then per layer  qkv (LN on load) -> self-attention -> o (+residual) -> cross q (LN on
// load) -> cross-attention -> cross o (+residual) -> fc1 (LN on load, activation) -> fc2 (+residual), then the
// vocabulary projection (final LN on load) with per-tile argmax and the pick: 3 + 8 L kernels. The residual stream x
// stays fp32; projections add into it in their epilogue and normalise it while staging their operand.
#include "common.cuh"

namespace b200dec_detail {
int linear_impl(const b200dec_weight* w, const void* a, int a_kind, const b200dec_norm* ln, int lda, int rows, void* out,
                int out_kind, int ldo, int act, int pdl, void* stream, const b200dec_ln_link* link,
                const KvPrefetch* pf);
int head_impl(const b200dec_weight* w, const void* a, int a_kind, const b200dec_norm* ln, int lda, int rows, float* pmax,
              int* pidx, float* logits, int pdl, void* stream);
int head_umma_impl(const b200dec_weight* w, const float* x, const void* xg, const float* stats, int stats_slots,
                   const b200dec_norm* ln, int lda, int rows, float* part_max, int32_t* part_idx, float* logits,
                   int32_t* status, int pdl, void* stream, int wait_limit, int withhold);
int embed_ln_impl(const int32_t* active, const int64_t* tok, const int32_t* pos, const void* embed,
                  const void* pos_table, int vocab, int max_pos, int slots, b200dec_norm ln0, b200dec_norm ln1,
                  float* x, void* hn, int hn_kind, int rows, int32_t* status, int pdl, void* stream,
                  const int32_t* cross_len, int seq, int frames, int32_t* sched_self, int32_t* sched_cross, void* x16,
                  const float* next_gamma, float* stats, int prefetch_keys);
int linear_passes(const b200dec_weight* w, int a_kind, bool ln, int rows);
int pick_impl(const float* part_max, const int32_t* part_idx, int partials, const int32_t* active, int rows, int dummy,
              int64_t* tok, int32_t* pos, uint8_t* finished, const int64_t* forced, int max_prompt,
              const int32_t* plen, const int32_t* limit, int64_t* out, int out_cols, int eos, int64_t* argmax,
              uint8_t* flags_host, int pdl, void* stream);
}  // namespace b200dec_detail

using namespace b200dec_detail;

#define B200_TRY(call)            \
  do {                            \
    const int rc_ = (call);       \
    if (rc_ != 0) return rc_;     \
  } while (0)
// a launch that belongs to one class of the step's kernels (b200dec_plan.classes)
#define B200_TRY_IN(cls, call) \
  do {                         \
    if (want & (cls)) B200_TRY(call); \
  } while (0)

extern "C" {

int b200dec_sizeof(int which) {
  switch (which) {
    case 0: return (int)sizeof(b200dec_weight);
    case 1: return (int)sizeof(b200dec_norm);
    case 2: return (int)sizeof(b200dec_layer);
    case 3: return (int)sizeof(b200dec_plan);
    case 4: return (int)sizeof(b200dec_ln_link);
  }
  return -1;
}

// Kernels one b200dec_step of `rows` rows launches: embedding, per layer six projections (a projection whose tile does
// not hold the rows goes in two passes) and two attention kernels, the vocabulary projection, the pick.
int b200dec_step_launches(const b200dec_plan* pl, int rows) {
  if (!pl || !pl->layer || rows < 1) return 0;
  const bool linked = pl->xh && pl->ln_stats && pl->a_kind == B200DEC_A_F16 && pl->layer[0].qkv.kind != B200DEC_W_BF16;
  const int ln_kind = linked ? B200DEC_A_F16_ROWS16 : pl->a_kind;
  int n = 2;  // embedding, pick
  for (int i = 0; i < pl->layers; ++i) {
    const b200dec_layer& ly = pl->layer[i];
    n += 2 + linear_passes(&ly.qkv, ln_kind, true, rows) + linear_passes(&ly.o, pl->a_kind, false, rows) +
         linear_passes(&ly.cq, ln_kind, true, rows) + linear_passes(&ly.co, pl->a_kind, false, rows) +
         linear_passes(&ly.fc1, ln_kind, true, rows) + linear_passes(&ly.fc2, pl->a_kind, false, rows);
  }
  n += is_umma_kind(pl->head.kind) ? 1 : linear_passes(&pl->head, pl->head_a_kind, true, rows);
  return n;
}

// Rows [row0, row0 + rows) of the step's batch as one chain of kernels. Every scratch buffer is indexed by row, so
// disjoint row ranges may run concurrently on different streams (the caller forks and joins them).
int b200dec_step_rows(const b200dec_plan* pl, int row0, int rows, void* stream) {
  B200_REQUIRE(pl && pl->layer && pl->layers >= 1, "step: null plan or no layers");
  B200_REQUIRE(rows >= 1 && row0 >= 0 && row0 + rows <= 128, "step: rows %d + %d outside 0..128", row0, rows);
  B200_REQUIRE(pl->heads * pl->head_dim == D_MODEL, "step: heads * head_dim must be %d", D_MODEL);
  B200_REQUIRE(pl->vocab == pl->head.n, "step: vocab %d vs head rows %d", pl->vocab, pl->head.n);
  B200_REQUIRE(!(pl->kv_int8 && pl->attn_ring), "step: the ring attention kernel reads bf16 caches only");
  const int hd = pl->heads * pl->head_dim;
  const int want = pl->classes ? pl->classes : 7;  // 1 embedding / vocabulary projection / pick, 2 projections, 4 attention
  // which launches carry the programmatic-dependent-launch attribute: bit 0 a projection (or the pick) that follows a
  // projection, bit 1 the attention kernels, bit 2 a projection that follows an attention kernel
  const int pdl = pl->pdl & 1, pdl_attn = (pl->pdl >> 1) & 1, pdl_after = (pl->pdl >> 2) & 1;
  const bool a16 = pl->a_kind == B200DEC_A_F16;
  const int ok_a = a16 ? B200DEC_OUT_F16 : B200DEC_OUT_F32;
  const float scale = 1.0f / sqrtf((float)pl->head_dim);
  const int ffn = pl->layer[0].fc1.n, partials = b200dec_head_partials(&pl->head);
  // this row range's share of every buffer
  const int32_t* active = pl->active + row0;
  float* x = pl->x + (size_t)row0 * D_MODEL;
  float* qkv = pl->qkv + (size_t)row0 * 3 * hd;
  float* cq = pl->cq + (size_t)row0 * hd;
  void* att = (char*)pl->att + (size_t)row0 * hd * (a16 ? 2 : 4);
  void* mid = (char*)pl->mid + (size_t)row0 * ffn * (a16 ? 2 : 4);
  float* attn_part = pl->attn_part ? pl->attn_part + b200dec_attention_scratch_floats(row0, pl->heads, pl->head_dim) : nullptr;
  int32_t* attn_count = pl->attn_count ? pl->attn_count + (size_t)row0 * pl->heads : nullptr;
  float* head_max = pl->head_max + (size_t)row0 * partials;
  int32_t* head_idx = pl->head_idx + (size_t)row0 * partials;
  float* logits = pl->logits ? pl->logits + (size_t)row0 * pl->vocab : nullptr;

  // The LayerNorm-folding projections stage an fp16 copy of the residual stream when the plan has one and the layer
  // projections are the kind that can (single fp16 operand, int8 or 2:4 weights, K slice <= 256); the projections that
  // update the stream (and the embedding) write that copy.
  void* xh = nullptr;
  if (pl->xh && pl->ln_stats && a16 && pl->layer[0].qkv.kind != B200DEC_W_BF16 &&
      b200dec_linear_fits(pl->layer[0].qkv.kind, B200DEC_A_F16_ROWS16, 1, pl->layer[0].qkv.warps, pl->layer[0].qkv.ksplit,
                          D_MODEL, rows) &&
      b200dec_linear_fits(pl->layer[0].cq.kind, B200DEC_A_F16_ROWS16, 1, pl->layer[0].cq.warps, pl->layer[0].cq.ksplit,
                          D_MODEL, rows) &&
      b200dec_linear_fits(pl->layer[0].fc1.kind, B200DEC_A_F16_ROWS16, 1, pl->layer[0].fc1.warps, pl->layer[0].fc1.ksplit,
                          D_MODEL, rows))
    xh = (char*)pl->xh + (size_t)row0 * D_MODEL * 2;
  const void* ln_src = xh ? xh : (const void*)x;
  const int ln_kind = xh ? B200DEC_A_F16_ROWS16 : pl->a_kind;
  // The statistics travel as partial sums, one slot per row and finishing CTA of the producer (the embedding: one).
  constexpr int STAT_SLOTS = 128;
  float* stats = xh ? pl->ln_stats + (size_t)row0 * STAT_SLOTS * 2 : nullptr;
  if (xh) {
    const b200dec_layer& l0 = pl->layer[0];
    B200_REQUIRE(b200dec_linear_stat_slots(&l0.o) <= STAT_SLOTS && b200dec_linear_stat_slots(&l0.co) <= STAT_SLOTS &&
                     b200dec_linear_stat_slots(&l0.fc2) <= STAT_SLOTS, "step: more finishing CTAs than statistic slots");
  }
  // the tcgen05 vocabulary projection takes the last fc2's rows the same way when its weight carries the folded vectors
  const bool head_linked = xh && is_umma_kind(pl->head.kind) && pl->head.ln_g && pl->head.ln_bias;
  auto producer = [&](const float* gamma) {
    b200dec_ln_link l{};
    l.status = pl->status, l.wait_limit = pl->wait_limit, l.withhold = (pl->withhold >> 1) & 1;
    if (xh && gamma) l.next_gamma = gamma, l.out16 = xh, l.stats_out = stats;
    return l;
  };
  auto reader = [&](int slots) {
    b200dec_ln_link l{};
    l.status = pl->status, l.wait_limit = pl->wait_limit, l.withhold = (pl->withhold >> 1) & 1;
    if (xh) l.stats_in = stats, l.stats_slots = slots;
    return l;
  };

  const auto attention = pl->attn_ring ? b200dec_attention_ring : b200dec_attention;
  // a large batch: the rows are ranked by length once (an extra CTA of the embedding kernel) and the attention
  // kernels pair long rows with short ones from the two tables
  const bool paired = !pl->attn_ring && pl->sched_self && pl->sched_cross && rows * pl->heads >= 512 && rows <= 256;
  int32_t* sched_self = paired ? pl->sched_self + 4 * row0 : nullptr;
  int32_t* sched_cross = paired ? pl->sched_cross + 4 * row0 : nullptr;

  // Prefetch of the attention launches' caches into L2 by the output projections (common.cuh, KvPrefetch): the budget
  // in keys per launch; one key of a row is 2 (key, value) x heads x vec_bytes bytes.
  const int vec_bytes = pl->head_dim * (pl->kv_int8 ? 1 : 2);
  const int prefetch_keys =
      paired && pl->kv_prefetch_mb > 0 ? (int)(((long long)pl->kv_prefetch_mb << 20) / (2LL * pl->heads * vec_bytes)) : 0;
  auto prefetch = [&](const int32_t* sched, const void* k, const void* v, int cap) {
    KvPrefetch f{};
    if (prefetch_keys > 0 && k && v)
      f = KvPrefetch{reinterpret_cast<const int4*>(sched), (const char*)k, (const char*)v, rows, pl->heads, cap, vec_bytes,
                     pl->slots};
    return f;
  };

  B200_TRY_IN(1, embed_ln_impl(active, pl->tok, pl->pos, pl->embed, pl->pos_table, pl->vocab, pl->max_pos, pl->slots,
                         pl->emb_ln, pl->layer[0].ln1, x, nullptr, B200DEC_OUT_F32, rows, pl->status, pdl, stream,
                         pl->cross_len, pl->seq, pl->frames, sched_self, sched_cross, xh, pl->layer[0].ln1.w, stats,
                         prefetch_keys));
  for (int i = 0; i < pl->layers; ++i) {
    const b200dec_layer& ly = pl->layer[i];
    // who wrote the operand and statistics each LayerNorm-folding projection reads: qkv <- embedding (1 slot) or the
    // previous layer's fc2; cross-q <- o; fc1 <- cross-o
    const b200dec_ln_link r1 = reader(i == 0 ? 1 : b200dec_linear_stat_slots(&pl->layer[i - 1].fc2)),
                          p2 = producer(ly.ln2.w), r2 = reader(b200dec_linear_stat_slots(&ly.o)),
                          p3 = producer(ly.ln3.w), r3 = reader(b200dec_linear_stat_slots(&ly.co)),
                          p1 = producer(i + 1 < pl->layers ? pl->layer[i + 1].ln1.w : head_linked ? pl->final_ln.w : nullptr);
    // what the two output projections start towards L2: this layer's cross caches, the next layer's self caches
    const KvPrefetch f_cross = prefetch(sched_cross, ly.cross_k, ly.cross_v, pl->frames);
    const KvPrefetch f_self = i + 1 < pl->layers ? prefetch(sched_self, pl->layer[i + 1].self_k, pl->layer[i + 1].self_v, pl->seq)
                                                 : KvPrefetch{};
    B200_TRY_IN(2, linear_impl(&ly.qkv, ln_src, ln_kind, &ly.ln1, D_MODEL, rows, qkv, B200DEC_OUT_F32, 3 * hd,
                         B200DEC_ACT_NONE, pdl, stream, &r1, nullptr));
    // The paired attention kernels read their two schedule entries before they wait for their predecessor, which is
    // sound while a kernel sits between the one that builds the schedule (the embedding) and them. With the
    // projections left out (classes) the first self-attention would follow the embedding directly and the two CTAs of
    // a pair could see different versions of an entry and disagree on their hand-off: it is then launched plainly.
    const int pdl_self = (i == 0 && !(want & 2)) ? 0 : pdl_attn;
    if (pl->kv_int8 && paired)
      B200_TRY_IN(4, b200dec_attention_paired_q8(1, sched_self, qkv, 3 * hd, ly.self_k, ly.self_v, ly.self_ks, ly.self_vs,
                                           pl->heads, pl->head_dim, pl->seq, scale, att, ok_a, rows, pdl_self, stream));
    else if (pl->kv_int8)
      B200_TRY_IN(4, b200dec_attention_q8(1, active, qkv, 3 * hd, ly.self_k, ly.self_v, ly.self_ks, ly.self_vs, pl->pos,
                                    pl->slots, pl->heads, pl->head_dim, pl->seq, scale, att, ok_a, rows, attn_part,
                                    attn_count, pl->status, pdl_self, stream));
    else if (paired)
      B200_TRY_IN(4, b200dec_attention_paired(1, sched_self, qkv, 3 * hd, ly.self_k, ly.self_v, pl->heads, pl->head_dim,
                                        pl->seq, scale, att, ok_a, rows, pdl_self, stream));
    else
      B200_TRY_IN(4, attention(1, active, qkv, 3 * hd, ly.self_k, ly.self_v, pl->pos, pl->slots, pl->heads,
                                 pl->head_dim, pl->seq, scale, att, ok_a, rows, attn_part, attn_count, pl->status,
                                 pdl_self, stream));
    B200_TRY_IN(2, linear_impl(&ly.o, att, pl->a_kind, nullptr, hd, rows, x, B200DEC_OUT_F32_ADD, D_MODEL, B200DEC_ACT_NONE,
                         pdl_after, stream, &p2, &f_cross));
    B200_TRY_IN(2, linear_impl(&ly.cq, ln_src, ln_kind, &ly.ln2, D_MODEL, rows, cq, B200DEC_OUT_F32, hd, B200DEC_ACT_NONE, pdl,
                         stream, &r2, nullptr));
    if (pl->kv_int8 && paired)
      B200_TRY_IN(4, b200dec_attention_paired_q8(0, sched_cross, cq, hd, (void*)ly.cross_k, (void*)ly.cross_v, ly.cross_ks,
                                           ly.cross_vs, pl->heads, pl->head_dim, pl->frames, scale, att, ok_a, rows,
                                           pdl_attn, stream));
    else if (pl->kv_int8)
      B200_TRY_IN(4, b200dec_attention_q8(0, active, cq, hd, (void*)ly.cross_k, (void*)ly.cross_v, ly.cross_ks, ly.cross_vs,
                                    pl->cross_len, pl->slots, pl->heads, pl->head_dim, pl->frames, scale, att, ok_a,
                                    rows, attn_part, attn_count, pl->status, pdl_attn, stream));
    else if (paired)
      B200_TRY_IN(4, b200dec_attention_paired(0, sched_cross, cq, hd, (void*)ly.cross_k, (void*)ly.cross_v, pl->heads,
                                        pl->head_dim, pl->frames, scale, att, ok_a, rows, pdl_attn, stream));
    else
      B200_TRY_IN(4, attention(0, active, cq, hd, (void*)ly.cross_k, (void*)ly.cross_v, pl->cross_len, pl->slots,
                                 pl->heads, pl->head_dim, pl->frames, scale, att, ok_a, rows, attn_part, attn_count,
                                 pl->status, pdl_attn, stream));
    B200_TRY_IN(2, linear_impl(&ly.co, att, pl->a_kind, nullptr, hd, rows, x, B200DEC_OUT_F32_ADD, D_MODEL, B200DEC_ACT_NONE,
                         pdl_after, stream, &p3, &f_self));
    B200_TRY_IN(2, linear_impl(&ly.fc1, ln_src, ln_kind, &ly.ln3, D_MODEL, rows, mid, ok_a, ffn, pl->act, pdl, stream, &r3,
                         nullptr));
    // the last layer's fc2 feeds the vocabulary projection
    B200_TRY_IN(2, linear_impl(&ly.fc2, mid, pl->a_kind, nullptr, ffn, rows, x, B200DEC_OUT_F32_ADD, D_MODEL,
                         B200DEC_ACT_NONE, pdl, stream, &p1, nullptr));
  }
  if (is_umma_kind(pl->head.kind))
    B200_TRY_IN(1, head_umma_impl(&pl->head, head_linked ? nullptr : x, head_linked ? xh : nullptr, stats,
                            b200dec_linear_stat_slots(&pl->layer[pl->layers - 1].fc2), &pl->final_ln, D_MODEL, rows,
                            head_max, head_idx, logits, pl->status, pdl, stream, pl->wait_limit, pl->withhold & 1));
  else
    B200_TRY_IN(1, head_impl(&pl->head, x, pl->head_a_kind, &pl->final_ln, D_MODEL, rows, head_max, head_idx, logits, pdl,
                       stream));
  B200_TRY_IN(1, pick_impl(head_max, head_idx, partials, active, rows, pl->slots, pl->tok, pl->pos, pl->finished, pl->forced,
                     pl->max_prompt, pl->plen, pl->limit, pl->out, pl->out_cols, pl->eos, pl->argmax, pl->flags_host, pdl,
                           stream));
  return 0;
}

int b200dec_step(const b200dec_plan* pl, int rows, void* stream) { return b200dec_step_rows(pl, 0, rows, stream); }

}  // extern "C"
