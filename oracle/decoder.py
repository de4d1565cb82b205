"""TEST INFRASTRUCTURE, not product code: fp32 numpy restatement of the reference decoder's token loop.

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs may import this package.

What it restates. The reference's GPU step (kernels/stream_decoder.py:176-199, kernels/csrc/decoder_ops.cu) is defined
as "the same text as transformers up to rounding" (server.py:24-25); the arithmetic itself lives in the third-party
package `transformers` (requirements.txt:4 pins >=5.4; 5.5.0 here), file
transformers/models/cohere_asr/modeling_cohere_asr.py:
  embedding + learned position + embedding LayerNorm      :386-401   (decoder_ops.cu:24-54)
  layer = x + SelfAttn(LN1 x); x + CrossAttn(LN2 x); x + MLP(LN3 x)   :258-294   (stream_decoder.py:179-196)
  attention = softmax(q k^T * head_dim^-0.5) v, fp32                   :73-96     (dec_attn.cuh:65-188)
  MLP = fc2(act(fc1 x)), act = ACT2FN[hidden_act]                       :46-58
  final LayerNorm, proj_out                                             :416, :553 (stream_decoder.py:173-174, 197)
  cross K/V = k_proj / v_proj of decoder.proj(memory)                   :386, cross-attention forward
                                                                         (stream_decoder.py:91-94, 229-232)
and the slot bookkeeping of one step is the reference's dec_pick (decoder_ops.cu:106-159), admit
(stream_decoder.py:241-263), set_active (:265-272) and reset (:216-222).

Pinning. No test in the reference repository holds a vector for this path ("parity unpinned" at the unit level there);
this restatement is pinned against transformers itself, run in the build container on the seed's weights:
tests/golden/decoder_*.npz (made by tests/golden/make_golden.py) and tests/test_oracle_decoder.py.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np

from . import packers

F32 = np.float32


def _erf(x: np.ndarray) -> np.ndarray:
    try:
        from scipy.special import erf  # vectorised, double precision inside
        return erf(x.astype(np.float64)).astype(F32)
    except Exception:  # pragma: no cover
        return np.vectorize(math.erf, otypes=[np.float64])(x).astype(F32)


def activation(name: str, x: np.ndarray) -> np.ndarray:
    if name == "relu":
        return np.maximum(x, 0)
    if name == "gelu":  # ACT2FN["gelu"] = the erf form
        return (0.5 * x * (1.0 + _erf(x * F32(1 / math.sqrt(2))))).astype(F32)
    raise ValueError(name)


def layer_norm(x: np.ndarray, w: np.ndarray, b: np.ndarray, eps: float) -> np.ndarray:
    x64 = x.astype(np.float64)
    mean = x64.mean(-1, keepdims=True)
    var = ((x64 - mean) ** 2).mean(-1, keepdims=True)
    return (((x64 - mean) / np.sqrt(var + eps)) * w + b).astype(F32)


def bf16_round(a: np.ndarray) -> np.ndarray:
    """fp32 -> nearest-even bfloat16 -> fp32 (the values a bf16 tensor holds)."""
    u = np.ascontiguousarray(a, dtype=F32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(F32).reshape(np.shape(a))


LINEARS = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "encoder_attn.q_proj",
           "encoder_attn.k_proj", "encoder_attn.v_proj", "encoder_attn.o_proj", "mlp.fc1", "mlp.fc2")


def effective_weights(state: dict, layers: int, mode: str = "fp32", tables: str = "fp32") -> dict:
    """fp32 weights the GPU path is defined to compute with, from a transformers-style state dict of fp32 arrays.

    mode: "fp32" as is; "bf16" every Linear weight rounded to bf16; "int8" every Linear weight of the decoding step
    (not the embeddings) replaced by q * s of quantize_rows (dec_w8.cu:4-5: "exactly those of the dequantized
    weights"); "int8_24" the same with mlp.fc1 / mlp.fc2 magnitude-pruned 2:4 first. The weights of the prefill
    (decoder.proj and the cross-attention k_proj / v_proj, which run once per request and not in the step) stay bf16
    in the int8 modes, as the reference keeps them (stream_decoder.py:91-94, 232). The three projections of
    self-attention are quantised as one fused (3d, d) matrix the way the reference fuses them (stream_decoder.py:56-57,
    87-90): rows are independent, so that equals quantising each alone. tables: "bf16" rounds the token and position
    tables to bf16 (how the GPU stores them); Linear biases and LayerNorm parameters stay fp32."""
    out = {k: np.asarray(v, dtype=F32) for k, v in state.items() if not k.startswith("model.encoder")}
    lin = [f"model.decoder.layers.{i}.{n}.weight" for i in range(layers) for n in LINEARS]
    lin += ["proj_out.weight", "model.decoder.proj.weight"]
    for k in lin:
        w = out[k]
        prefill = k == "model.decoder.proj.weight" or ".encoder_attn.k_proj." in k or ".encoder_attn.v_proj." in k
        if mode == "bf16" or (prefill and mode in ("int8", "int8_24")):
            out[k] = bf16_round(w)
        elif mode in ("int8", "int8_24"):
            if mode == "int8_24" and (".mlp.fc1." in k or ".mlp.fc2." in k):
                w = packers.prune_24_magnitude(w)
            out[k] = packers.dequantize(*packers.quantize_rows(w))
        elif mode != "fp32":
            raise ValueError(mode)
    if tables == "bf16":
        for k in ("model.decoder.embed_tokens.weight", "model.decoder.pos_emb.weight"):
            out[k] = bf16_round(out[k])
    return out


@dataclass
class OracleConfig:
    layers: int
    heads: int
    head_dim: int
    act: str
    eps: float = 1e-5
    pad: int = 2
    eos: int = 3

    @classmethod
    def of(cls, cfg) -> "OracleConfig":
        return cls(cfg.num_hidden_layers, cfg.num_attention_heads, cfg.head_dim, cfg.hidden_act,
                   getattr(cfg, "layer_norm_eps", 1e-5), cfg.pad_token_id, cfg.eos_token_id)


def kv_int8(a: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """The reference's int8 cache format (kernels/csrc/dec_attn.cuh:46-63, decoder_ops.cu:190-203): per vector along
    the last axis scale = absmax / 127 (1 for a zero vector), q = rint(clamp(x * (1 / scale), +-127)), all in fp32,
    rint = half to even. Returns (q int8, scale fp32 with the last axis kept at length 1)."""
    a = np.asarray(a, dtype=F32)
    mx = np.abs(a).max(-1, keepdims=True).astype(F32)
    sc = np.where(mx > 0, (mx / F32(127)).astype(F32), F32(1)).astype(F32)
    inv = (F32(1) / sc).astype(F32)
    q = np.rint(np.clip((a * inv).astype(F32), F32(-127), F32(127)))
    return q.astype(np.int8), sc


def kv_int8_round(a: np.ndarray) -> np.ndarray:
    """What an int8 cache gives back for a vector that was rounded to bf16 and then quantised: q * scale in fp32."""
    q, sc = kv_int8(bf16_round(a))
    return (q.astype(F32) * sc).astype(F32)


class OracleDecoder:
    """One decoding step over explicit per-sequence caches. kv_round: "bf16" rounds keys and values to bf16 when they
    enter a cache (what a bf16 KV cache holds); "int8" stores the int8 form of the bf16-rounded vector (kv_int8) and,
    as the reference does, attends a row's new key and value in the step that appends them as the bf16 values; None
    keeps fp32."""

    def __init__(self, weights: dict, cfg: OracleConfig, kv_round: str | None = None):
        self.w, self.cfg, self.kv_round = weights, cfg, kv_round
        self.scale = F32(cfg.head_dim ** -0.5)

    def _p(self, name):
        return self.w[name]

    def _lin(self, x, prefix):
        return (x @ self.w[prefix + ".weight"].T + self.w[prefix + ".bias"]).astype(F32)

    def _ln(self, x, prefix):
        return layer_norm(x, self.w[prefix + ".weight"], self.w[prefix + ".bias"], self.cfg.eps)

    def _store(self, a):
        if self.kv_round == "int8":
            return kv_int8_round(a)
        return bf16_round(a) if self.kv_round == "bf16" else a.astype(F32)

    def cross_kv(self, memory: np.ndarray) -> list[tuple[np.ndarray, np.ndarray]]:
        """memory (T, enc_dim) -> per layer (K, V) each (H, T, D)."""
        c = self.cfg
        m = self._lin(np.asarray(memory, dtype=F32), "model.decoder.proj")
        out = []
        for i in range(c.layers):
            p = f"model.decoder.layers.{i}.encoder_attn"
            k = self._lin(m, p + ".k_proj").reshape(-1, c.heads, c.head_dim).transpose(1, 0, 2)
            v = self._lin(m, p + ".v_proj").reshape(-1, c.heads, c.head_dim).transpose(1, 0, 2)
            out.append((self._store(k), self._store(v)))
        return out

    def new_self_cache(self):
        return [([], []) for _ in range(self.cfg.layers)]

    def _attend(self, q, k, v):
        """q (H, D); k, v (H, n, D) -> (H*D,)"""
        s = np.einsum("hd,hnd->hn", q.astype(np.float64), k.astype(np.float64)) * float(self.scale)
        s -= s.max(-1, keepdims=True)
        p = np.exp(s)
        p /= p.sum(-1, keepdims=True)
        return np.einsum("hn,hnd->hd", p, v.astype(np.float64)).astype(F32).reshape(-1)

    def step(self, tok: np.ndarray, pos: np.ndarray, self_caches: list, cross: list, taps: dict | None = None):
        """Feed token tok[r] at position pos[r] for every row r. self_caches[r] = list per layer of ([K rows], [V
        rows]) grown in place; cross[r] = cross_kv(memory_r). Returns logits (B, V) fp32."""
        c, B = self.cfg, len(tok)
        E, P = self._p("model.decoder.embed_tokens.weight"), self._p("model.decoder.pos_emb.weight")
        x = self._ln((E[tok] + P[pos]).astype(F32), "model.decoder.embedding_layernorm")
        for i in range(c.layers):
            p = f"model.decoder.layers.{i}"
            h = self._ln(x, p + ".input_layernorm")
            q, k, v = (self._lin(h, f"{p}.self_attn.{n}_proj") for n in "qkv")
            a = np.empty_like(x)
            for r in range(B):
                ks, vs = self_caches[r][i]
                assert len(ks) == pos[r], "self cache length must equal the position being fed"
                kn, vn = k[r].reshape(c.heads, c.head_dim), v[r].reshape(c.heads, c.head_dim)
                ks.append(self._store(kn))
                vs.append(self._store(vn))
                if self.kv_round == "int8":  # this step sees the new pair before quantisation
                    kk = np.stack(ks[:-1] + [bf16_round(kn)], 1)
                    vv = np.stack(vs[:-1] + [bf16_round(vn)], 1)
                else:
                    kk, vv = np.stack(ks, 1), np.stack(vs, 1)
                a[r] = self._attend(q[r].reshape(c.heads, c.head_dim), kk, vv)
            x = x + self._lin(a, p + ".self_attn.o_proj")
            h = self._ln(x, p + ".post_attention_layernorm")
            q = self._lin(h, p + ".encoder_attn.q_proj")
            for r in range(B):
                ck, cv = cross[r][i]
                a[r] = self._attend(q[r].reshape(c.heads, c.head_dim), ck, cv)
            x = x + self._lin(a, p + ".encoder_attn.o_proj")
            h = self._ln(x, p + ".final_layernorm")
            mid = activation(c.act, self._lin(h, p + ".mlp.fc1"))
            x = x + self._lin(mid, p + ".mlp.fc2")
            if taps is not None:
                taps[f"x{i}"] = x.copy()
        h = self._ln(x, "model.decoder.norm")
        if taps is not None:
            taps["final"] = h.copy()
        return self._lin(h, "proj_out")


def argmax_first(logits: np.ndarray) -> np.ndarray:
    """First index of the maximum, NaN never winning (decoder_ops.cu:118-147; torch.argmax on CPU)."""
    lg = np.where(np.isnan(logits), -np.inf, logits)
    return lg.argmax(-1)


class StreamOracle:
    """The reference StreamDecoder's host API and slot semantics on the CPU (stream_decoder.py:65-276), for parity of
    whole decoding runs and as the decoder behind scheduler tests. record=True keeps, per step, the list
    (slot, position fed, logits row, un-forced argmax)."""

    BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 80, 96, 112, 128)

    def __init__(self, weights: dict, cfg: OracleConfig, slots: int = 128, max_new_tokens: int = 448,
                 max_prompt: int = 16, frames: int = 451, buckets=None, kv_round: str | None = None,
                 eos: int | None = None, record: bool = False):
        self.dec = OracleDecoder(weights, cfg, kv_round)
        self.cfg = cfg
        self.slots, self.dummy = slots, slots
        self.buckets = tuple(b for b in (buckets or self.BUCKETS) if b <= slots)
        self.max_new_tokens, self.max_prompt = max_new_tokens, max_prompt
        self.seq = max_prompt + max_new_tokens + 1
        self.frames = frames
        self.eos = cfg.eos if eos is None else eos
        self.pad = cfg.pad
        S = slots
        self.tok = np.full(S + 1, self.pad, np.int64)
        self.pos = np.zeros(S + 1, np.int32)
        self.plen = np.ones(S + 1, np.int32)
        self.limit = np.zeros(S + 1, np.int32)
        self.cross_len = np.ones(S + 1, np.int32)
        self.finished = np.ones(S + 1, np.uint8)
        self.forced = np.full((S + 1, max_prompt), self.pad, np.int64)
        self.out = np.full((S + 1, self.seq + 1), self.pad, np.int64)
        self.flags = np.ones(S + 1, np.uint8)
        self.active = np.full(max(self.buckets), S, np.int32)
        self.cross = [None] * (S + 1)
        self.self_kv = [self.dec.new_self_cache() for _ in range(S + 1)]
        self.record = [] if record else None
        self.steps = 0

    def bucket(self, rows: int) -> int:
        return next(b for b in self.buckets if b >= rows)

    def reset(self) -> None:
        self.finished[:] = 1
        self.pos[:] = 0
        self.cross_len[:] = 1
        self.active[:] = self.dummy

    def fill_cross(self, hidden: np.ndarray, lengths: list[int], slots: list[int]) -> None:
        """hidden (sum(lengths), enc_dim) packed frames (stream_decoder.py:229-239)."""
        at = 0
        for n, s in zip(lengths, slots):
            assert 1 <= n <= self.frames
            self.cross[s] = self.dec.cross_kv(hidden[at:at + n])
            at += n

    def admit(self, slots, prompts, frames, max_new=None) -> None:
        """stream_decoder.py:241-263"""
        for i, s in enumerate(slots):
            p = np.asarray(prompts[i], dtype=np.int64)
            assert 1 <= len(p) <= self.max_prompt
            self.forced[s] = self.pad
            self.forced[s, :len(p)] = p
            self.out[s] = self.pad
            self.out[s, :self.max_prompt] = self.forced[s]
            self.tok[s], self.pos[s], self.plen[s] = p[0], 0, len(p)
            self.limit[s] = len(p) - 1 + (max_new[i] if max_new else self.max_new_tokens)
            self.cross_len[s] = frames[i]
            self.finished[s] = 0
            self.flags[s] = 0
            self.self_kv[s] = self.dec.new_self_cache()

    def set_active(self, slots) -> int:
        b = self.bucket(max(1, len(slots)))
        self.active[:b] = self.dummy
        self.active[:len(slots)] = slots
        return b

    def step(self, bucket: int) -> None:
        """One replay: stream_decoder.py:176-199 with dec_pick's bookkeeping (decoder_ops.cu:106-159). Rows on the
        dummy slot are not computed here (their results are discarded by the reference too, :112-113); a finished
        row recomputes its last position and changes nothing (:151)."""
        rows = [int(s) for s in self.active[:bucket] if s != self.dummy]
        if rows:
            tok, pos = self.tok[rows], self.pos[rows]
            caches = []
            for s in rows:  # a finished row re-feeds its position: drop the entry it appended last time
                for ks, vs in self.self_kv[s]:
                    del ks[self.pos[s]:], vs[self.pos[s]:]
                caches.append(self.self_kv[s])
            logits = self.dec.step(tok, pos, caches, [self.cross[s] for s in rows])
            arg = argmax_first(logits)
            for r, s in enumerate(rows):
                if self.record is not None:
                    self.record.append((self.steps, s, int(self.pos[s]), logits[r].copy(), int(arg[r])))
                if self.finished[s]:
                    continue
                at = int(self.pos[s]) + 1
                in_prompt = at < self.plen[s]
                nt = int(self.forced[s, at]) if in_prompt else int(arg[r])
                self.out[s, at] = nt
                self.tok[s], self.pos[s] = nt, at
                self.finished[s] = 1 if (not in_prompt and (nt == self.eos or at >= self.limit[s])) else 0
        self.flags[:] = self.finished
        self.steps += 1


def state_to_numpy(model) -> dict:
    """fp32 numpy state dict of a torch model (decoder + head only)."""
    return {k: v.detach().to("cpu").float().numpy() for k, v in model.state_dict().items()
            if not k.startswith("model.encoder")}
