"""Greedy decoding with continuous batching on one B200: the reference's StreamDecoder API over the b200dec kernels.

Drop-in for kernels/stream_decoder.py:65-276 of the reference: the same constructor arguments, attributes (`device`,
`out`, `flags`, `stream`, `eos`, `max_new_tokens`, `buckets`, `slots`, `dummy`) and methods (`fill_cross`, `admit`,
`set_active`, `step`, `reset`, `bucket`) with the same meaning, so the reference's Pipeline (kernels/pipeline.py) can
drive it unchanged. Row r of a step works on slot active[r]; rows past the live ones point at the dummy slot; a step
is one CUDA-graph launch per bucket of row counts; the prompt is fed by the steps themselves as forced tokens; a row
that ends sets its flag in pinned host memory from the step's last kernel (no copy node in the graph).

What differs underneath: every kernel is hand-written CUDA for sm_100a behind a C-ABI (include/b200dec.h), there is no
Triton and no cuBLAS on the step; `int8=True` quantises every projection of the step (also o, cross q and cross o; the
prefill's projections keep bf16 weights), `ffn_sparse=True` additionally stores fc1/fc2 2:4, `fp16_weights=True` is the
16-bit mode on the same kernels (the bf16 weight values as fp16); the residual stream is fp32; heads x head_dim may
be 8 x 128 or 16 x 64 and the feed-forward activation ReLU or GELU (read from model.config). The wide projections
(qkv, fc1) and the vocabulary projection run on tcgen05 / tensor memory, in buckets of up to `umma_above_rows` rows on
the register-dequantising mma.sync kernel from a second packing of the same weights.
"""

from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import native as nv
from .packing import PackedLinear, dequantized, pack_linear

ACTS = {"relu": nv.ACT_RELU, "gelu": nv.ACT_GELU}


def _fp32(t: torch.Tensor) -> torch.Tensor:
    return t.detach().float().contiguous()


class _Layer:
    """One decoder layer as the step's kernels read it: six packed projections (q, k and v fused into one, as the
    reference fuses them, kernels/stream_decoder.py:56-57) and the three LayerNorms in fp32. The projections that
    follow a LayerNorm (qkv, cross-q, fc1) are packed together with that norm's folded vectors."""

    # name -> (modules whose weights are stacked, index of the LayerNorm folded into it or None, feed-forward?)
    SPEC = {"qkv": (("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"), 0, False),
            "o": (("self_attn.o_proj",), None, False),
            "cq": (("encoder_attn.q_proj",), 1, False),
            "co": (("encoder_attn.o_proj",), None, False),
            "fc1": (("mlp.fc1",), 2, True),
            "fc2": (("mlp.fc2",), None, True)}

    UMMA_KIND = {nv.W_INT8: nv.W_INT8_UMMA, nv.W_F16: nv.W_F16_UMMA, nv.W_INT8_24: nv.W_INT8_24_UMMA}

    def __init__(self, layer, kind: int, ffn_kind: int, a_kind: int, max_rows: int, keep_reference: bool,
                 umma: frozenset = frozenset(), small_rows: int = 0):
        self.small = {}  # name -> the mma.sync packing of a tcgen05 projection, for buckets of up to small_rows rows
        self.norms = [(_fp32(m.weight), _fp32(m.bias), float(m.eps)) for m in
                      (layer.input_layernorm, layer.post_attention_layernorm, layer.final_layernorm)]
        for name, (paths, norm, ffn) in self.SPEC.items():
            mods = [layer.get_submodule(p) for p in paths]
            k = ffn_kind if ffn else kind
            w, b = torch.cat([_fp32(m.weight) for m in mods]), torch.cat([_fp32(m.bias) for m in mods])
            ln = None if norm is None else self.norms[norm][:2]
            if name in umma and k in self.UMMA_KIND:  # on the tcgen05 kernel
                if small_rows:
                    self.small[name] = pack_linear(w, b, k, False, a_kind=a_kind, max_rows=small_rows, ln=ln)
                k = self.UMMA_KIND[k]
            setattr(self, name, pack_linear(w, b, k, keep_reference, a_kind=a_kind, max_rows=max_rows, ln=ln))

    def projections(self) -> list[PackedLinear]:
        return [getattr(self, name) for name in self.SPEC]


class _PrefillWeight:
    """One projection of the cross-attention prefill (fill_cross; the reference's two F.linear, kernels/
    stream_decoder.py:232) for csrc/prefill_gemm.cu: the weight rounded to bf16 in the kernel's tile image, the bias
    fp32. Output channels are padded with zero rows to a multiple of 256."""

    def __init__(self, w: torch.Tensor, b: torch.Tensor):
        n, k = w.shape
        assert k % 64 == 0, "prefill: the input width must be a multiple of 64"
        self.n, self.k = -(-n // 256) * 256, k
        wb = torch.zeros(self.n, k, dtype=torch.bfloat16, device=w.device)
        wb[:n] = w.detach().to(torch.bfloat16)
        self.image = torch.empty(self.n * k * 2, dtype=torch.uint8, device=w.device)
        nv.check(nv.lib().b200dec_prefill_tile_weight(nv.ptr(wb), self.n, k, nv.ptr(self.image), nv.stream_ptr()))
        torch.cuda.current_stream().synchronize()
        self.bias = torch.zeros(self.n, device=w.device)
        self.bias[:n] = b.detach().float()


class StreamDecoder:
    BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 80, 96, 112, 128)

    def __init__(self, model, slots: int = 128, max_new_tokens: int = 448, max_prompt: int = 16,
                 max_audio_s: float = 36.0, buckets=None, int8: bool = False, *, ffn_sparse: bool = False,
                 eos: int | None = None, record: bool = False, pdl: bool | int = 7, graphs: bool = True,
                 head_split: bool = True, keep_reference: bool = False, chains: int = 1, attn_ring: bool = False,
                 head_umma: bool = True, kv_int8: bool = False, proj_umma: bool | str = True,
                 kv_prefetch_mb: int = 0, device_sched: bool = False, fp16_weights: bool = False,
                 umma_above_rows: int = 16,
                 _packed: tuple | None = None):
        """model: a CohereAsrForConditionalGeneration-shaped module on a CUDA device (see synth.synthetic_model).
        int8: weight-only int8 with per-output-channel scales on every projection (fp16 activations, fp32
        accumulation); else bf16 weights with the fp32 activations split into two bf16 halves, or with fp16_weights
        the fp16 image of those bf16 weights (packing.fp16_image) on the int8 mode's pipeline: fp16 activations, the
        LayerNorms folded through the fp16 copy of the residual stream, twice the weight bytes of int8 and no
        quantisation error. ffn_sparse: fc1/fc2
        magnitude-pruned 2:4 and stored compressed (needs int8). eos: overrides config.eos_token_id (-1: never end on
        a token). record: keep the last step's logits and every slot's un-forced argmax (teacher forcing, tests).
        pdl: which of the step's kernels launch programmatically after their predecessor (bits: 1 a projection after a
        projection, 2 the attention kernels, 4 a projection after attention; True = 1, False = 0). graphs: capture one CUDA graph per bucket
        (False: launch the kernels directly, for debugging). chains: a step's rows are split into up to this many
        independent kernel chains that run concurrently (parallel branches of the graph), so that one chain's
        attention overlaps the others' projections; results do not depend on it. attn_ring: use the persistent
        bulk-copy attention kernel (csrc/attention_ring.cu) instead of the one-CTA-per-(row, head) kernel.
        kv_prefetch_mb: the projections between two attention launches start up to this many MB of the next launch's
        keys and values on their way into L2 (0: off). device_sched: the active list lives on the device: `admit`
        appends to it, every step drops the rows that ended and leaves the live count in `live` (pinned), so a
        scheduler never calls set_active after an eviction. umma_above_rows: the tcgen05 layer projections serve the
        buckets of more than this many rows, the smaller buckets run a second, mma.sync packing of the same weights
        (0: tcgen05 in every bucket)."""
        nv.lib()  # fail now, loudly, if the CUDA library is missing
        assert not ffn_sparse or int8, "2:4 feed-forward weights are int8"
        assert not (fp16_weights and int8), "fp16_weights is a mode of its own beside int8"
        cfg = model.config
        dev = model.device if _packed else model.model.decoder.embed_tokens.weight.device
        assert dev.type == "cuda", "StreamDecoder needs the model on a CUDA device: there is no CPU path"
        self.device = dev
        self.buckets = tuple(b for b in (buckets or self.BUCKETS) if b <= slots)
        self.model, self.max_new_tokens = (None if _packed else model), max_new_tokens
        self.h, self.d, self.width = cfg.num_attention_heads, cfg.head_dim, cfg.hidden_size
        assert self.width == 1024 and (self.h, self.d) in ((8, 128), (16, 64)), "1024 wide, 8 x 128 or 16 x 64 heads"
        self.eos = cfg.eos_token_id if eos is None else eos
        self.pad = cfg.pad_token_id
        self.scale = self.d ** -0.5
        self.int8, self.ffn_sparse, self.pdl, self.use_graphs = int8, ffn_sparse, pdl, graphs
        self.attn_ring = bool(attn_ring)
        self.kv_prefetch_mb, self.device_sched = int(kv_prefetch_mb), bool(device_sched)
        assert not (self.device_sched and chains > 1), "the device-side active list goes with a single chain"
        self.act, self._act_name, self._cfg_eos = ACTS[cfg.hidden_act], cfg.hidden_act, cfg.eos_token_id
        self.fp16_weights = bool(fp16_weights)
        kind = nv.W_INT8 if int8 else nv.W_F16 if fp16_weights else nv.W_BF16
        half_rows = bool(int8 or fp16_weights)  # activations travel as fp16 rows
        ffn_kind = nv.W_INT8_24 if ffn_sparse else kind
        self.a_kind = nv.A_F16 if half_rows else nv.A_F32_SPLIT
        self.head_a_kind = nv.A_F16 if (fp16_weights or (int8 and not head_split)) else nv.A_F32_SPLIT
        bm = max(self.buckets)
        with torch.cuda.device(dev):
            # proj_umma: the dense int8 projections that run on the tcgen05 kernel of csrc/linear_umma.cu: True = qkv and
            # fc1 (the two with enough multiply per CTA to gain; the narrow ones and fc2 measured 1-2 % slower there
            # than on mma.sync), "all", or a comma-separated subset of qkv,o,cq,co,fc1,fc2
            # (fp16 weights: none by default; with qkv and fc1 there the 64-row step measured 0.550 ms against 0.514)
            names = ("qkv,fc1" if int8 else "") if proj_umma is True else \
                "qkv,o,cq,co,fc1,fc2" if proj_umma == "all" else (proj_umma or "")
            umma = frozenset(n for n in names.split(",") if n) if half_rows else frozenset()
            # umma_above_rows: those projections run on tcgen05 in buckets of more than this many rows; the smaller
            # buckets use a second, mma.sync packing of the same weights (at 1-16 rows the 64-row tensor-memory tile and
            # its set-up cost 2.3 us per launch more than the 16-row mma.sync tile: 0.287 -> 0.252 ms per step at 1 row,
            # 0.336 -> 0.311 at 16, equal at 24, tcgen05 ahead from 32). 0: tcgen05 in every bucket, one packing.
            small = [b for b in self.buckets if b <= umma_above_rows]
            self._small_rows = max(small) if (small and umma) else 0
            self._pack_options = dict(int8=bool(int8), fp16_weights=bool(fp16_weights), ffn_sparse=bool(ffn_sparse),
                                      head_split=bool(head_split), head_umma=bool(head_umma),
                                      proj_umma=",".join(sorted(umma)), max_rows=bm, small_rows=self._small_rows)
            if _packed:
                self._load_packed(*_packed)
            else:
                self._pack_from_model(model, kind, ffn_kind, bm, keep_reference, umma, head_umma)
            self.vocab, self.max_pos = self.embed.shape[0], self.pos_table.shape[0]
            assert self.proj.n == self.width and self.cross.n == len(self.layers) * 2 * self.width
            L, S = len(self.layers), slots
            self.slots, self.dummy = S, S
            self.max_prompt = max_prompt
            self.seq = max_prompt + max_new_tokens + 1
            assert self.seq <= self.max_pos, "positions exceed the learned position table"
            self.frames = int(model.model.encoder._get_subsampling_output_length(
                torch.tensor([int(max_audio_s * 100) + 1])).item())
            # kv_int8: keys and values as int8 with one fp32 scale per head vector, the format of the reference's int8
            # mode (stream_decoder.py:102-115); otherwise bf16
            self.kv_int8 = bool(kv_int8)
            assert not (self.kv_int8 and attn_ring), "the ring attention kernel reads bf16 caches only"
            # KV caches: (layer, slot incl. the dummy, head, position, dim); int8 caches carry one fp32 scale per vector
            kv_dtype = torch.int8 if self.kv_int8 else torch.bfloat16
            for name, cap in (("self", self.seq), ("cross", self.frames)):
                for part in "kv":
                    setattr(self, f"{name}_{part}", torch.zeros(L, S + 1, self.h, cap, self.d, device=dev, dtype=kv_dtype))
                    setattr(self, f"{name}_{part}s",
                            torch.ones(L, S + 1, self.h, cap, device=dev) if self.kv_int8 else None)
            # slot state, one entry per slot and one for the dummy; names, types and initial values are those of the
            # reference's StreamDecoder (kernels/stream_decoder.py:116-131), which is what its callers read
            i32 = dict(device=dev, dtype=torch.int32)
            state = dict(cross_len=(torch.int32, (), 1), tok=(torch.long, (), self.pad), pos=(torch.int32, (), 0),
                         plen=(torch.int32, (), 1), limit=(torch.int32, (), 0), finished=(torch.uint8, (), 1),
                         forced=(torch.long, (max_prompt,), self.pad), out=(torch.long, (self.seq + 1,), self.pad))
            for name, (dtype, tail, value) in state.items():
                setattr(self, name, torch.full((S + 1, *tail), value, device=dev, dtype=dtype))
            self.active = torch.full((bm,), S, **i32)
            self.status = torch.zeros(1, **i32)
            self.n_active = torch.zeros(1, **i32)  # device_sched: live rows at the front of `active`
            self.live = torch.zeros(1, dtype=torch.int32).pin_memory()  # its copy after the newest finished step
            # host -> device staging: packed admission records / row lists through a ring of pinned buffers
            self._rec_ints = nv.lib().b200dec_admit_record_ints(max_prompt)
            self._admit_cap = max(bm, 16)
            self.admit_buf = torch.zeros(self._admit_cap * self._rec_ints, **i32)
            self._ring = [(torch.zeros(self._admit_cap * self._rec_ints, dtype=torch.int32).pin_memory(),
                           torch.cuda.Event()) for _ in range(8)]
            self._ring_at = 0
            adt = torch.float16 if self.a_kind == nv.A_F16 else torch.float32
            f32 = dict(device=dev, dtype=torch.float32)
            self.x = torch.zeros(bm, self.width, **f32)
            self.qkv = torch.zeros(bm, 3 * self.width, **f32)
            self.cq = torch.zeros(bm, self.width, **f32)
            self.att = torch.zeros(bm, self.width, device=dev, dtype=adt)
            self.ffn = self.layers[0].fc1.n
            self.mid = torch.zeros(bm, self.ffn, device=dev, dtype=adt)
            lib = nv.lib()
            self.attn_part = torch.zeros(lib.b200dec_attention_scratch_floats(bm, self.h, self.d), **f32)
            self.attn_count = torch.zeros(bm * self.h, **i32)
            self.head_partials = lib.b200dec_head_partials(C.byref(self.head.struct()))
            self.head_max = torch.zeros(bm, self.head_partials, **f32)
            self.head_idx = torch.zeros(bm, self.head_partials, **i32)
            # the step's rows ranked by length (self / cross), rebuilt by every step for the paired attention kernel
            # the residual stream times the next LayerNorm's gamma as fp16, and the rows' partial sums (one slot per
            # finishing CTA of the producer): what the LayerNorm-folding projections stage (int8, 2:4 and fp16 weights)
            self.xh = torch.zeros(bm, self.width, device=dev, dtype=torch.float16) if half_rows else None
            self.ln_stats = torch.zeros(bm, 128, 2, device=dev) if half_rows else None
            self.sched_self = torch.zeros(bm, 4, **i32)
            self.sched_cross = torch.zeros(bm, 4, **i32)
            self.logits = torch.zeros(bm, self.vocab, **f32) if record else None
            self.argmax = torch.zeros(S + 1, device=dev, dtype=torch.long) if record else None
            # host side: the end flags after each step (pinned, written by the step itself)
            self.flags = torch.ones(S + 1, dtype=torch.uint8).pin_memory()
            self.graphs: dict[int, torch.cuda.CUDAGraph] = {}
            self.stream = torch.cuda.Stream(device=dev, priority=-1)
            self.chains = max(1, int(chains))
            self.side_streams = [torch.cuda.Stream(device=dev, priority=-1) for _ in range(self.chains - 1)]
            self._build_plan()
            self._select_layers(min(self.buckets))
            self.launches_per_step = lib.b200dec_step_launches(C.byref(self.plan), min(self.buckets))
            self.weight_bytes = sum(p.stream_bytes() for ly in self.layers for p in ly.projections()) + \
                self.head.stream_bytes()
            if graphs:
                self._capture()
            else:
                self.reset()
                self.stream.synchronize()

    # ---- weights: packed from a model, or loaded as packed ---------------------------------------------------------

    def _pack_from_model(self, model, kind, ffn_kind, bm, keep_reference, umma, head_umma) -> None:
        dec = model.model.decoder
        self.embed = dec.embed_tokens.weight.detach().to(torch.bfloat16).contiguous()
        self.pos_table = dec.pos_emb.weight.detach().to(torch.bfloat16).contiguous()
        ln = lambda m: (_fp32(m.weight), _fp32(m.bias), float(m.eps))  # noqa: E731
        self.emb_ln, self.final_ln = ln(dec.embedding_layernorm), ln(dec.norm)
        self.layers = [_Layer(layer, kind, ffn_kind, self.a_kind, bm, keep_reference, umma, self._small_rows)
                       for layer in dec.layers]
        head_kind = kind
        if head_umma and kind in (nv.W_INT8, nv.W_F16) and self.embed.shape[0] % 128 == 0:
            head_kind = nv.W_INT8_UMMA if self.int8 else nv.W_F16_UMMA
        self.head = pack_linear(model.proj_out.weight, model.proj_out.bias, head_kind, keep_reference,
                                a_kind=self.head_a_kind, ln=self.final_ln[:2], max_rows=bm)
        # prefill: cross K/V of all layers as one (L * 2 * d, d) matrix behind the encoder projection; these run once
        # per request, not in the step, and keep bf16 weights in every mode, as the reference does
        # (kernels/stream_decoder.py:91-94, 232)
        self.proj = _PrefillWeight(_fp32(dec.proj.weight), _fp32(dec.proj.bias))
        self.cross = _PrefillWeight(
            torch.cat([_fp32(w) for layer in dec.layers
                       for w in (layer.encoder_attn.k_proj.weight, layer.encoder_attn.v_proj.weight)]),
            torch.cat([_fp32(b) for layer in dec.layers
                       for b in (layer.encoder_attn.k_proj.bias, layer.encoder_attn.v_proj.bias)]))

    def _load_packed(self, manifest: dict, tensors: dict) -> None:
        """The weights exactly as save_packed wrote them (same tiling, same bits): nothing is re-quantised."""
        if manifest["pack_options"] != self._pack_options:
            raise ValueError(f"packed with {manifest['pack_options']}, asked for {self._pack_options}")
        t = {k: v.to(self.device) for k, v in tensors.items()}
        self.embed, self.pos_table = t["embed"], t["pos_table"]
        eps = manifest["eps"]
        self.emb_ln, self.final_ln = ((t[n + ".w"], t[n + ".b"], eps[n]) for n in ("emb_ln", "final_ln"))

        def packed(name: str) -> PackedLinear:
            m = manifest["projections"][name]
            return PackedLinear(m["kind"], m["n"], m["k"], t[name + ".tiled"], t.get(name + ".meta"), t.get(name + ".scale"),
                                t.get(name + ".bias"), m["warps"], m["ksplit"], ln_g=t.get(name + ".ln_g"),
                                ln_bias=t.get(name + ".ln_bias"))
        self.layers = []
        for i in range(manifest["layers"]):
            ly = object.__new__(_Layer)
            ly.norms = [(t[f"layer{i}.ln{j}.w"], t[f"layer{i}.ln{j}.b"], eps[f"layer{i}.ln{j}"]) for j in (1, 2, 3)]
            for name in _Layer.SPEC:
                setattr(ly, name, packed(f"layer{i}.{name}"))
            ly.small = {name: packed(f"layer{i}.{name}.small") for name in _Layer.SPEC
                        if f"layer{i}.{name}.small" in manifest["projections"]}
            self.layers.append(ly)
        self.head = packed("head")
        for name in ("proj", "cross"):
            w = object.__new__(_PrefillWeight)
            w.image, w.bias = t[f"prefill.{name}.image"], t[f"prefill.{name}.bias"]
            w.n, w.k = manifest["prefill"][name]
            setattr(self, name, w)

    def save_packed(self, path: str) -> str:
        """Writes the packed weights (every tensor of packed_tensors(), as the kernels read them) with a manifest: the
        model's configuration, the packing options, every projection's kind and tile, and the SHA-256 of the lot.
        StreamDecoder.from_packed(path) gives a decoder with the same bits without the original model. Returns the
        digest."""
        digest = self.weights_digest()
        proj = {f"layer{i}.{n}": getattr(ly, n) for i, ly in enumerate(self.layers) for n in _Layer.SPEC}
        proj.update({f"layer{i}.{n}.small": p for i, ly in enumerate(self.layers) for n, p in ly.small.items()})
        proj["head"] = self.head
        eps = {"emb_ln": self.emb_ln[2], "final_ln": self.final_ln[2]}
        eps.update({f"layer{i}.ln{j + 1}": ly.norms[j][2] for i, ly in enumerate(self.layers) for j in range(3)})
        manifest = dict(
            format=1, sha256=digest, layers=len(self.layers), eps=eps, pack_options=self._pack_options,
            config=dict(num_attention_heads=self.h, head_dim=self.d, hidden_size=self.width, hidden_act=self._act_name,
                        eos_token_id=self._cfg_eos, pad_token_id=self.pad),
            projections={k: dict(kind=p.kind, n=p.n, k=p.k, warps=p.warps, ksplit=p.ksplit) for k, p in proj.items()},
            prefill=dict(proj=(self.proj.n, self.proj.k), cross=(self.cross.n, self.cross.k)))
        torch.save(dict(manifest=manifest, tensors={k: v.detach().cpu() for k, v in self.packed_tensors().items()}), path)
        return digest

    @classmethod
    def from_packed(cls, path: str, device: torch.device | str = "cuda", **kw) -> "StreamDecoder":
        """A decoder from a file written by save_packed: the manifest's digest is checked against the loaded bytes
        before anything else. kw: the run-time arguments of the constructor (slots, max_new_tokens, max_prompt,
        max_audio_s, buckets, eos, record, pdl, kv_int8, device_sched, ...); the packing options come from the file
        (the largest bucket must be the one the weights were tiled for)."""
        from types import SimpleNamespace
        from .synth import _EncoderStub
        blob = torch.load(path, map_location="cpu", weights_only=True)
        man = blob["manifest"]
        if man.get("format") != 1:
            raise ValueError(f"{path}: unknown packed-weight format {man.get('format')}")
        shim = SimpleNamespace(config=SimpleNamespace(**man["config"]), device=torch.device(device),
                               model=SimpleNamespace(encoder=_EncoderStub()))
        if shim.device.index is None:
            shim.device = torch.device("cuda", torch.cuda.current_device())
        po = man["pack_options"]
        if "umma_above_rows" in kw:
            raise ValueError("umma_above_rows is a packing option: it comes from the file")
        self = cls(shim, int8=po["int8"], fp16_weights=po.get("fp16_weights", False), ffn_sparse=po["ffn_sparse"],
                   head_split=po["head_split"], umma_above_rows=po.get("small_rows", 0),
                   head_umma=po["head_umma"], proj_umma=po["proj_umma"] or False, _packed=(man, blob["tensors"]), **kw)
        if self.weights_digest() != man["sha256"]:
            raise ValueError(f"{path}: the packed weights do not match the manifest's SHA-256")
        return self

    @classmethod
    def from_checkpoint(cls, path: str, device: torch.device | str = "cuda", dtype: torch.dtype | None = None,
                        **kw) -> "StreamDecoder":
        """A decoder from a Cohere Transcribe checkpoint directory (config.json + *.safetensors, single or sharded):
        only the decoder's tensors are read, the encoder is never built (checkpoint.load_decoder). The reference gets
        the same weights by loading the whole model through transformers (server.py:264-267). dtype: convert the
        stored floating-point tensors first (None: as stored). kw: the constructor's arguments."""
        from .checkpoint import load_decoder
        dev = torch.device(device)
        if dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        return cls(load_decoder(path, dtype).to(dev), **kw)

    # ---- the step ------------------------------------------------------------------------------------------------

    def _build_plan(self) -> None:
        L = len(self.layers)

        def layer_structs(small: bool):
            structs = (nv.Layer * L)()
            for i, ly in enumerate(self.layers):
                s = structs[i]
                s.ln1, s.ln2, s.ln3 = (nv.norm(*n) for n in ly.norms)
                for name in _Layer.SPEC:
                    setattr(s, name, ((ly.small.get(name) if small else None) or getattr(ly, name)).struct())
                s.self_k, s.self_v = nv.ptr(self.self_k[i]), nv.ptr(self.self_v[i])
                s.cross_k, s.cross_v = nv.ptr(self.cross_k[i]), nv.ptr(self.cross_v[i])
                if self.kv_int8:
                    s.self_ks, s.self_vs = nv.ptr(self.self_ks[i]), nv.ptr(self.self_vs[i])
                    s.cross_ks, s.cross_vs = nv.ptr(self.cross_ks[i]), nv.ptr(self.cross_vs[i])
            return structs
        self._layer_structs = layer_structs(False)
        # the same layers with the mma.sync packings of the tcgen05 projections, for buckets up to _small_rows rows
        self._layer_structs_small = layer_structs(True) if self._small_rows else None
        p = nv.Plan()
        p.layers, p.heads, p.head_dim, p.act = L, self.h, self.d, self.act
        p.slots, p.seq, p.frames, p.vocab = self.slots, self.seq, self.frames, self.vocab
        p.max_prompt, p.out_cols, p.pad, p.eos = self.max_prompt, self.out.shape[1], self.pad, self.eos
        p.a_kind, p.max_pos, p.head_a_kind, p.pdl = self.a_kind, self.max_pos, self.head_a_kind, int(self.pdl)
        p.attn_ring, p.kv_int8 = int(self.attn_ring), int(self.kv_int8)
        p.embed, p.pos_table = nv.ptr(self.embed), nv.ptr(self.pos_table)
        p.emb_ln, p.final_ln = nv.norm(*self.emb_ln), nv.norm(*self.final_ln)
        p.layer = C.cast(self._layer_structs, C.POINTER(nv.Layer))
        p.head = self.head.struct()
        for name in ("active", "tok", "pos", "plen", "limit", "cross_len", "finished", "forced", "out", "status", "x",
                     "qkv", "cq", "att", "mid", "attn_part", "attn_count", "head_max", "head_idx",
                     "xh", "ln_stats", "sched_self", "sched_cross", "logits", "argmax"):
            setattr(p, name, nv.ptr(getattr(self, name)))
        p.kv_prefetch_mb = int(self.kv_prefetch_mb)
        # pinned host memory is addressable from the device: a row that ends sets its byte of `flags` from the pick
        # kernel (admit() clears it on the host, as the reference does)
        p.flags_host = self.flags.data_ptr()
        self.plan = p

    def _select_layers(self, b: int) -> None:
        """Points the plan at the layer packings bucket b runs on (a captured graph keeps what it was captured with)."""
        small = self._layer_structs_small is not None and b <= self._small_rows
        self.plan.layer = C.cast(self._layer_structs_small if small else self._layer_structs, C.POINTER(nv.Layer))

    def _step(self, b: int) -> None:
        """Bucket b's kernels on the current stream (reference: _step, stream_decoder.py:176-199; the end flags reach
        `flags` from the pick kernel)."""
        self._select_layers(b)
        ranges = self.row_ranges(b)
        if len(ranges) == 1:
            nv.check(nv.lib().b200dec_step(C.byref(self.plan), b, nv.stream_ptr()))
        else:
            # independent chains over disjoint rows on forked streams: one chain's attention (HBM-bound) overlaps the
            # others' projections (latency-bound); the fork and the join are events, so a capture records them as
            # parallel branches of the graph
            main = torch.cuda.current_stream()
            fork = torch.cuda.Event()
            fork.record(main)
            for (r0, n), side in zip(ranges, [main] + self.side_streams):
                if side is not main:
                    side.wait_event(fork)
                nv.check(nv.lib().b200dec_step_rows(C.byref(self.plan), r0, n, side.cuda_stream))
                if side is not main:
                    done = torch.cuda.Event()
                    done.record(side)
                    main.wait_event(done)
        if self.device_sched:  # rows that ended leave the device's active list; the host learns the live count
            nv.check(nv.lib().b200dec_compact_active(C.byref(self.plan), b, nv.ptr(self.n_active), self.live.data_ptr(),
                                                     int(self.pdl) & 1, nv.stream_ptr()))

    def launches(self, rows: int) -> int:
        """Kernels one step of `rows` rows launches (summed over its chains)."""
        count = nv.lib().b200dec_step_launches
        self._select_layers(rows)
        return sum(count(C.byref(self.plan), n) for _, n in self.row_ranges(rows)) + (1 if self.device_sched else 0)

    def row_ranges(self, b: int) -> list[tuple[int, int]]:
        """The (first row, rows) of the concurrent chains a step of b rows is split into: at most `chains` ranges of
        whole 8-row tiles."""
        c = max(1, min(self.chains, b // 8))
        per = ((b + c - 1) // c + 7) // 8 * 8 if c > 1 else b
        out, r0 = [], 0
        while r0 < b:
            out.append((r0, min(per, b - r0)))
            r0 += per
        return out

    @torch.no_grad()
    def _capture(self) -> None:
        """One CUDA graph per bucket, largest first so that the graphs share one memory pool sized by the largest.
        Each bucket runs once directly before its capture: that sets the kernels' attributes and surfaces launch
        errors where they can be reported."""
        pool = torch.cuda.graph_pool_handle()
        with torch.cuda.device(self.device), torch.cuda.stream(self.stream):
            for rows in sorted(self.buckets, reverse=True):
                self._step(rows)
                self.stream.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, pool=pool, stream=self.stream):
                    self._step(rows)
                self.graphs[rows] = graph
        self.reset()
        self.stream.synchronize()
        self.check_status()

    def capture_classes(self, mask: int) -> None:
        """A timing aid: from now on a step launches only the kernels of `mask` (b200dec_plan.classes: 1 embedding,
        vocabulary projection and pick, 2 layer projections, 4 attention; 0 = the whole step again). The graphs are
        captured anew and every slot is reset; results of partial steps are meaningless."""
        self.plan.classes = int(mask)
        if self.use_graphs:
            self._capture()
        else:
            self.reset()

    def reset(self) -> None:
        """Every slot free and every row on the dummy slot (on the decoder stream). The dummy keeps position 0 and
        one frame, so the rows that pad a bucket always have a key to attend."""
        with torch.cuda.stream(self.stream):
            for t, v in ((self.finished, 1), (self.pos, 0), (self.cross_len, 1), (self.active, self.dummy),
                         (self.status, 0), (self.attn_count, 0), (self.n_active, 0)):
                t.fill_(v)
        self.flags.fill_(1)  # the host's copy (the steps write it through; nothing is in flight at a reset)

    def check_status(self) -> None:
        """Synchronises the decoder stream and raises if a kernel met an index outside its tables (the kernels clamp
        the index, set a bit and go on, so the context stays usable)."""
        self.stream.synchronize()
        st = int(self.status.item())
        if st:
            names = [n for n, bit in (("out-of-range token id", nv.ST_TOKEN_RANGE),
                                      ("out-of-range position", nv.ST_POS_RANGE),
                                      ("out-of-range frame count", nv.ST_FRAMES_RANGE),
                                      ("out-of-range slot", nv.ST_SLOT_RANGE),
                                      ("a bounded wait inside a kernel ran out", nv.ST_TIMEOUT)) if st & bit]
            raise nv.NativeError("decoder kernels reported: " + ", ".join(names))

    # ---- host side -----------------------------------------------------------------------------------------------
    # Everything the host sends per call is packed into one pinned staging buffer and crosses in one asynchronous
    # copy; the slot fields are then written by one kernel (csrc/slots.cu). Same effects as the reference's methods
    # (kernels/stream_decoder.py:226-276).

    def bucket(self, rows: int) -> int:
        """The smallest captured row count that holds `rows` rows."""
        for b in self.buckets:
            if b >= rows:
                return b
        raise ValueError(f"{rows} rows exceed the largest bucket {self.buckets[-1]}")

    def _stage(self, values: np.ndarray, dst: torch.Tensor, stream: torch.cuda.Stream | None = None) -> None:
        """int32 values -> dst (device int32, at least as long) through the pinned ring, on `stream` (default: the
        decoder stream)."""
        stream = stream or self.stream
        n = int(values.size)
        buf, ev = self._ring[self._ring_at]
        self._ring_at = (self._ring_at + 1) % len(self._ring)
        ev.synchronize()  # the copy that last used this buffer (several calls ago) has long finished
        buf.numpy()[:n] = values.reshape(-1)
        with torch.cuda.stream(stream):
            dst[:n].copy_(buf[:n], non_blocking=True)
            ev.record(stream)

    @torch.no_grad()
    def fill_cross(self, hidden: torch.Tensor, lengths: list[int], slots: list[int]) -> None:
        """Cross-attention keys and values of packed encoder frames (sum(lengths), enc_dim), piece i = lengths[i]
        frames for slots[i], into the slot caches; on the current stream (the caller orders the decoder stream after
        it, as with the reference's method). Two tcgen05 products, the second writing the caches itself."""
        m = int(hidden.shape[0])
        if not (len(lengths) == len(slots) and m == sum(lengths) and hidden.shape[1] == self.proj.k):
            raise ValueError("fill_cross: hidden must hold sum(lengths) rows of the encoder width, one length per slot")
        if not all(1 <= n <= self.frames for n in lengths) or not all(0 <= s < self.slots for s in slots):
            raise ValueError(f"fill_cross: 1..{self.frames} frames per piece, slots 0..{self.slots - 1}")
        if m == 0:
            return
        lib, cur = nv.lib(), torch.cuda.current_stream()
        x = hidden.float().contiguous()
        pieces = np.zeros((len(slots), 4), np.int32)
        pieces[:, 0] = np.concatenate([[0], np.cumsum(lengths[:-1])])
        pieces[:, 1], pieces[:, 2] = lengths, slots
        table = torch.empty(pieces.size, dtype=torch.int32, device=self.device)
        if pieces.size <= self._ring[0][0].numel():
            self._stage(pieces, table, cur)
        else:
            table.copy_(torch.from_numpy(pieces.reshape(-1)))
        img = lambda k: torch.empty(lib.b200dec_prefill_rows_bytes(m, k) + 1024, dtype=torch.uint8, device=self.device)  # noqa: E731
        aligned = lambda t: t.data_ptr() + (-t.data_ptr()) % 1024  # noqa: E731
        a0, a1 = img(self.proj.k), img(self.proj.n)
        s = cur.cuda_stream
        nv.check(lib.b200dec_prefill_pack_rows(nv.ptr(x), m, self.proj.k, x.shape[1], aligned(a0), s))
        nv.check(lib.b200dec_prefill_gemm(aligned(a0), m, self.proj.k, nv.ptr(self.proj.image), nv.ptr(self.proj.bias),
                                          self.proj.n, 0, aligned(a1), None, 0, None, None, None, None, 0, 0, 0, 0, 0,
                                          nv.ptr(self.status), s))
        nv.check(lib.b200dec_prefill_gemm(aligned(a1), m, self.cross.k, nv.ptr(self.cross.image), nv.ptr(self.cross.bias),
                                          self.cross.n, 2 if self.kv_int8 else 1, None, nv.ptr(table), len(slots),
                                          nv.ptr(self.cross_k), nv.ptr(self.cross_v), nv.ptr(self.cross_ks),
                                          nv.ptr(self.cross_vs), len(self.layers), self.slots + 1, self.h, self.d,
                                          self.frames, nv.ptr(self.status), s))
        for t in (x, table, a0, a1):
            t.record_stream(cur)

    def admit(self, slots: list[int], prompts: list, frames: list[int], max_new: list[int] | None = None) -> None:
        """Start decoding in `slots`: each gets its prompt (fed token by token as forced choices), its number of
        encoder frames and its new-token budget (max_new_tokens when not given). On the decoder stream."""
        n = len(slots)
        budgets = list(max_new) if max_new else [self.max_new_tokens] * n
        if not (len(prompts) == len(frames) == len(budgets) == n):
            raise ValueError("admit: one prompt, frame count and budget per slot")
        rec = np.full((n, self._rec_ints), self.pad, np.int32)
        for i, (s, p, f, m) in enumerate(zip(slots, prompts, frames, budgets)):
            if isinstance(p, torch.Tensor):
                p = p.detach().cpu().numpy()
            p = np.asarray(p, dtype=np.int64).reshape(-1)
            if not (0 <= s < self.slots and 1 <= p.size <= self.max_prompt and 1 <= f <= self.frames
                    and 1 <= m <= self.max_new_tokens):
                raise ValueError(f"admit: slot {s}, prompt of {p.size}, {f} frames, {m} new tokens out of range")
            rec[i, :4] = (s, p.size, m, f)
            rec[i, 4:4 + p.size] = p
        torch.cuda.nvtx.range_push("b200dec.admit")
        for i0 in range(0, n, self._admit_cap):  # more requests than the staging buffer holds: several launches
            part = rec[i0:i0 + self._admit_cap]
            self._stage(part, self.admit_buf)
            nv.check(nv.lib().b200dec_admit(C.byref(self.plan), nv.ptr(self.admit_buf), len(part),
                                            nv.ptr(self.n_active) if self.device_sched else None, max(self.buckets),
                                            self.stream.cuda_stream))
        self.flags.numpy()[list(slots)] = 0
        torch.cuda.nvtx.range_pop()

    def set_active(self, slots: list[int]) -> int:
        """The rows of the next steps = these slots, padded with the dummy slot to a bucket; returns the bucket."""
        b = self.bucket(max(1, len(slots)))
        rows = np.full(b + 1, self.dummy, np.int32)
        rows[:len(slots)] = slots
        rows[b] = len(slots)
        self._stage(rows[:b], self.active)
        if self.device_sched:
            self._stage(rows[b:], self.n_active)
        return b

    def step(self, bucket: int) -> None:
        """One decoding step of `bucket` rows on the decoder stream (a graph replay)."""
        torch.cuda.nvtx.range_push("b200dec.step")
        with torch.cuda.stream(self.stream):
            if self.use_graphs:
                self.graphs[bucket].replay()
            else:
                self._step(bucket)
        torch.cuda.nvtx.range_pop()

    # ---- identity of the packed weights -----------------------------------------------------------------------------

    def packed_tensors(self) -> dict[str, torch.Tensor]:
        """Every tensor the kernels read as a weight (tiled projections, scales, biases, folded LayerNorm vectors,
        tables, norms, prefill images), by name, in a fixed order."""
        out: dict[str, torch.Tensor] = {"embed": self.embed, "pos_table": self.pos_table}
        for name, (w, b, _) in (("emb_ln", self.emb_ln), ("final_ln", self.final_ln)):
            out[name + ".w"], out[name + ".b"] = w, b
        packs = [(f"layer{i}.{n}", getattr(ly, n)) for i, ly in enumerate(self.layers)
                 for n in ("qkv", "o", "cq", "co", "fc1", "fc2")] + [("head", self.head)]
        packs += [(f"layer{i}.{n}.small", p) for i, ly in enumerate(self.layers) for n, p in ly.small.items()]
        for name, p in packs:
            for field in ("tiled", "meta", "scale", "bias", "ln_g", "ln_bias"):
                t = getattr(p, field)
                if t is not None:
                    out[f"{name}.{field}"] = t
        for i, ly in enumerate(self.layers):
            for j, (w, b, _) in enumerate(ly.norms):
                out[f"layer{i}.ln{j + 1}.w"], out[f"layer{i}.ln{j + 1}.b"] = w, b
        for name, p in (("prefill.proj", self.proj), ("prefill.cross", self.cross)):
            out[name + ".image"], out[name + ".bias"] = p.image, p.bias
        return out

    def weights_digest(self) -> str:
        """SHA-256 over the packed weights (names, shapes, dtypes and bytes as the kernels read them). Replicas of a
        data-parallel job compare it before they start (dataparallel.check_identical): the same bits on every GPU."""
        import hashlib
        h = hashlib.sha256()
        for name, t in self.packed_tensors().items():
            h.update(f"{name}|{tuple(t.shape)}|{t.dtype}|".encode())
            h.update(t.detach().contiguous().view(torch.uint8).cpu().numpy().tobytes())
        return h.hexdigest()

    # ---- accounting ------------------------------------------------------------------------------------------------

    def step_bytes(self, positions, frames, rows: int | None = None) -> int:
        """Algorithmic HBM bytes of one step whose live rows are at `positions` with `frames` encoder frames each
        (rows: the bucket, counting padding rows on the dummy slot as position 0 / 1 frame): every projection's
        weights once, each row's keys and values of both attentions in all layers, the appended key and value, the
        two embedding rows."""
        L, d = len(self.layers), self.width
        pad = (rows or len(positions)) - len(positions)
        kv = sum((int(p) + 1) + int(t) for p, t in zip(positions, frames)) + pad * 2
        n = len(positions) + pad
        # bytes per cached or appended vector element: 2 (bf16), or 1 + 4 / D (int8 and its share of the vector's scale)
        b_kv = 1 + 4 / self.d if self.kv_int8 else 2
        return int(self.weight_bytes + L * 2 * d * b_kv * kv + n * L * 2 * d * b_kv + n * 2 * d * 2)
