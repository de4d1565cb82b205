// One decoding step as a sequence of kernel launches on the caller's stream (capturable into a CUDA graph):
// embed + 2 LayerNorms, then per layer  qkv -> self-attention -> o (+residual) -> LN -> cross q -> cross-attention ->
// cross o (+residual) -> LN -> fc1 (+act) -> fc2 (+residual) -> LN, then the vocabulary projection with per-tile
// argmax and the pick. The residual stream x stays fp32; projections add into it in their epilogue.
#include "common.cuh"

namespace b200dec_detail {
int linear_impl(const b200dec_weight* w, const void* a, int a_kind, int lda, int rows, void* out, int out_kind,
                int ldo, int act, int pdl, void* stream);
int head_impl(const b200dec_weight* w, const void* a, int a_kind, int lda, int rows, float* pmax, int* pidx,
              float* logits, int pdl, void* stream);
int embed_ln_impl(const int32_t* active, const int64_t* tok, const int32_t* pos, const void* embed,
                  const void* pos_table, int vocab, int max_pos, int slots, b200dec_norm ln0, b200dec_norm ln1, float* x,
                  void* hn, int hn_kind, int rows, int32_t* status, int pdl, void* stream);
int layer_norm_impl(const float* x, b200dec_norm ln, void* hn, int hn_kind, int rows, int pdl, void* stream);
int pick_impl(const float* part_max, const int32_t* part_idx, int partials, const int32_t* active, int rows, int dummy,
              int64_t* tok, int32_t* pos, uint8_t* finished, const int64_t* forced, int max_prompt,
              const int32_t* plen, const int32_t* limit, int64_t* out, int out_cols, int eos, int64_t* argmax, int pdl,
              void* stream);
}  // namespace b200dec_detail

using namespace b200dec_detail;

#define B200_TRY(call)            \
  do {                            \
    const int rc_ = (call);       \
    if (rc_ != 0) return rc_;     \
  } while (0)

extern "C" {

int b200dec_step_launches(const b200dec_plan* plan, int rows) {
  (void)rows;
  return plan ? 3 + 11 * plan->layers : 0;
}

int b200dec_step(const b200dec_plan* pl, int rows, void* stream) {
  B200_REQUIRE(pl && pl->layer && pl->layers >= 1, "step: null plan or no layers");
  B200_REQUIRE(rows >= 1 && rows <= 128, "step: rows %d outside 1..128", rows);
  B200_REQUIRE(pl->heads * pl->head_dim == D_MODEL, "step: heads * head_dim must be %d", D_MODEL);
  B200_REQUIRE(pl->vocab == pl->head.n, "step: vocab %d vs head rows %d", pl->vocab, pl->head.n);
  const int hd = pl->heads * pl->head_dim, pdl = pl->pdl;
  const int ok_a = pl->a_kind == B200DEC_A_F16 ? B200DEC_OUT_F16 : B200DEC_OUT_F32;
  const int ok_head = pl->head_a_kind == B200DEC_A_F16 ? B200DEC_OUT_F16 : B200DEC_OUT_F32;
  const float scale = 1.0f / sqrtf((float)pl->head_dim);
  const int ffn = pl->layer[0].fc1.n;

  B200_TRY(embed_ln_impl(pl->active, pl->tok, pl->pos, pl->embed, pl->pos_table, pl->vocab, pl->max_pos, pl->slots,
                         pl->emb_ln, pl->layer[0].ln1, pl->x, pl->hn, ok_a, rows, pl->status, pdl, stream));
  for (int i = 0; i < pl->layers; ++i) {
    const b200dec_layer& ly = pl->layer[i];
    const bool last = i + 1 == pl->layers;
    B200_TRY(linear_impl(&ly.qkv, pl->hn, pl->a_kind, D_MODEL, rows, pl->qkv, B200DEC_OUT_F32, 3 * hd,
                         B200DEC_ACT_NONE, pdl, stream));
    B200_TRY(b200dec_attention(1, pl->active, pl->qkv, 3 * hd, ly.self_k, ly.self_v, pl->pos, pl->slots, pl->heads,
                               pl->head_dim, pl->seq, scale, pl->att, ok_a, rows, pl->attn_part, pl->attn_count,
                               pl->status, pdl, stream));
    B200_TRY(linear_impl(&ly.o, pl->att, pl->a_kind, hd, rows, pl->x, B200DEC_OUT_F32_ADD, D_MODEL, B200DEC_ACT_NONE,
                         pdl, stream));
    B200_TRY(layer_norm_impl(pl->x, ly.ln2, pl->hn, ok_a, rows, pdl, stream));
    B200_TRY(linear_impl(&ly.cq, pl->hn, pl->a_kind, D_MODEL, rows, pl->cq, B200DEC_OUT_F32, hd, B200DEC_ACT_NONE, pdl,
                         stream));
    B200_TRY(b200dec_attention(0, pl->active, pl->cq, hd, (void*)ly.cross_k, (void*)ly.cross_v, pl->cross_len,
                               pl->slots, pl->heads, pl->head_dim, pl->frames, scale, pl->att, ok_a, rows,
                               pl->attn_part, pl->attn_count, pl->status, pdl, stream));
    B200_TRY(linear_impl(&ly.co, pl->att, pl->a_kind, hd, rows, pl->x, B200DEC_OUT_F32_ADD, D_MODEL,
                         B200DEC_ACT_NONE, pdl, stream));
    B200_TRY(layer_norm_impl(pl->x, ly.ln3, pl->hn, ok_a, rows, pdl, stream));
    B200_TRY(linear_impl(&ly.fc1, pl->hn, pl->a_kind, D_MODEL, rows, pl->mid, ok_a, ffn, pl->act, pdl, stream));
    B200_TRY(linear_impl(&ly.fc2, pl->mid, pl->a_kind, ffn, rows, pl->x, B200DEC_OUT_F32_ADD, D_MODEL,
                         B200DEC_ACT_NONE, pdl, stream));
    if (last)
      B200_TRY(layer_norm_impl(pl->x, pl->final_ln, pl->hn_head, ok_head, rows, pdl, stream));
    else
      B200_TRY(layer_norm_impl(pl->x, pl->layer[i + 1].ln1, pl->hn, ok_a, rows, pdl, stream));
  }
  const int partials = b200dec_head_partials(&pl->head);
  B200_TRY(head_impl(&pl->head, pl->hn_head, pl->head_a_kind, D_MODEL, rows, pl->head_max, pl->head_idx, pl->logits,
                     pdl, stream));
  B200_TRY(pick_impl(pl->head_max, pl->head_idx, partials, pl->active, rows, pl->slots, pl->tok, pl->pos,
                     pl->finished, pl->forced, pl->max_prompt, pl->plen, pl->limit, pl->out, pl->out_cols, pl->eos,
                     pl->argmax, pdl, stream));
  return 0;
}

}  // extern "C"
