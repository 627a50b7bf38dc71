"""Typed configuration of the Sezazen decoder, read from its config.json.

The file describes the model layer by layer: `layers[i]` gives the layer's `type` (its mixer), the
mixer's sizes (`mixer`) and its feed-forward (`mlp`, or null for none); `loop` names a range of layers
whose layers are applied repeatedly (one set of weights, several passes); `embedding.scale`, `norm.eps`, `vocab`, `width`
and `max_positions` are the model's own.  Every size and every constant that the file gives is read
from it; what the design fixes (the sink's score of zero, the squared-ReLU experts, the tied output
head, the learned position vectors) is stated in `plan()`.

Tensor names: `embed`, `pos`, `loop.in`, `loop.step`, `final.norm`, and per layer `l<i>.norm1`,
`l<i>.norm2`, `l<i>.mix.{q,k,v,o}`, `l<i>.mlp.{gate,up,down}` (dense) or `l<i>.mlp.router`,
`l<i>.mlp.e<j>.{up,down}`, `l<i>.mlp.shared.{up,down}` (mixture of experts); linear weights `[out, in]`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .registry import register_architecture
from .specs import BlockSpec, ConfigError, JunctionCall, LayerCall, ModelPlan, PartSpec, WeightBinding

#: every softmax of the design has a sink of this score: exp(0) = 1 joins the sum of exponentials
SINK_LOGIT = 0.0


def _need(d, key, where):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key `{where}{key}` is missing")
    return d[key]


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int                  # size of a query and a key head
    vdim: int                 # size of a value head
    scale: float              # scores are (q . k) * scale


@dataclass(frozen=True)
class DenseMlp:
    ff: int


@dataclass(frozen=True)
class MoeMlp:
    experts: int
    top: int
    expert_ff: int
    shared_ff: int            # 0: no shared expert


@dataclass(frozen=True)
class SezazenLayer:
    type: str
    mixer: AttentionMixer
    mlp: object               # DenseMlp | MoeMlp | None


@dataclass(frozen=True)
class Loop:
    start: int
    stop: int
    times: int


@register_architecture("Sezazen")
@dataclass(frozen=True)
class SezazenConfig:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    embedding_scale: float
    layers: tuple
    loop: Optional[Loop] = None
    eos_token_id: Optional[tuple] = None

    MIXERS = ("attention",)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict) -> "SezazenConfig":
        layers = []
        for i, L in enumerate(_need(raw, "layers", "")):
            at = f"layers[{i}]."
            kind = _need(L, "type", at)
            if kind not in cls.MIXERS:
                raise ConfigError(f"config.json: {at}type {kind!r} is not a mixer of this design (known: {', '.join(cls.MIXERS)})")
            m = _need(L, "mixer", at)
            mixer = AttentionMixer(heads=int(_need(m, "heads", at + "mixer.")), kv_heads=int(_need(m, "kv_heads", at + "mixer.")),
                                   dim=int(_need(m, "dim", at + "mixer.")), vdim=int(_need(m, "vdim", at + "mixer.")),
                                   scale=float(_need(m, "scale", at + "mixer.")))
            f = L.get("mlp")
            if f is None:
                mlp = None
            else:
                fk = _need(f, "kind", at + "mlp.")
                if fk == "dense":
                    mlp = DenseMlp(ff=int(_need(f, "ff", at + "mlp.")))
                elif fk == "moe":
                    r = _need(f, "router", at + "mlp.")
                    shared = f.get("shared")
                    mlp = MoeMlp(experts=int(_need(r, "experts", at + "mlp.router.")), top=int(_need(r, "top", at + "mlp.router.")),
                                 expert_ff=int(_need(_need(f, "expert", at + "mlp."), "ff", at + "mlp.expert.")),
                                 shared_ff=int(_need(shared, "ff", at + "mlp.shared.")) if shared else 0)
                else:
                    raise ConfigError(f"config.json: {at}mlp.kind {fk!r} is unknown (dense, moe)")
            layers.append(SezazenLayer(kind, mixer, mlp))
        lp = raw.get("loop")
        loop = None
        if lp:
            loop = Loop(int(_need(lp, "start", "loop.")), int(_need(lp, "stop", "loop.")), int(_need(lp, "times", "loop.")))
        eos = raw.get("eos_token_id")
        if isinstance(eos, int):
            eos = (eos,)
        elif eos is not None:
            eos = tuple(int(x) for x in eos)
        cfg = cls(vocab=int(_need(raw, "vocab", "")), width=int(_need(raw, "width", "")),
                  max_positions=int(_need(raw, "max_positions", "")),
                  norm_eps=float(_need(_need(raw, "norm", ""), "eps", "norm.")),
                  embedding_scale=float(_need(_need(raw, "embedding", ""), "scale", "embedding.")),
                  layers=tuple(layers), loop=loop, eos_token_id=eos)
        cfg.validate()
        return cfg

    def validate(self):
        c = self
        for k, v in {"vocab": c.vocab, "width": c.width, "max_positions": c.max_positions}.items():
            if v <= 0:
                raise ConfigError(f"`{k}` must be positive, got {v}")
        if not c.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if not c.layers:
            raise ConfigError("a model needs at least one layer")
        for i, L in enumerate(c.layers):
            m = L.mixer
            if min(m.heads, m.kv_heads, m.dim, m.vdim) < 1:
                raise ConfigError(f"layers[{i}].mixer: heads, kv_heads, dim and vdim must be positive")
            if m.heads % m.kv_heads:
                raise ConfigError(f"layers[{i}].mixer: {m.heads} heads are no multiple of {m.kv_heads} kv_heads")
            if isinstance(L.mlp, DenseMlp) and L.mlp.ff < 1:
                raise ConfigError(f"layers[{i}].mlp.ff must be positive")
            if isinstance(L.mlp, MoeMlp):
                f = L.mlp
                if f.experts < 1 or not 1 <= f.top <= f.experts:
                    raise ConfigError(f"layers[{i}].mlp.router: top {f.top} must lie in 1..experts ({f.experts})")
                if f.expert_ff < 1 or f.shared_ff < 0:
                    raise ConfigError(f"layers[{i}].mlp: expert and shared sizes must be positive")
        if c.loop is not None:
            lp = c.loop
            if not 0 <= lp.start < lp.stop <= len(c.layers):
                raise ConfigError(f"loop: layers {lp.start}..{lp.stop - 1} are not a range of the model's {len(c.layers)}")
            if lp.times < 1:
                raise ConfigError("loop.times must be at least 1")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        layers = []
        for L in self.layers:
            m = L.mixer
            if L.mlp is None:
                mlp = None
            elif isinstance(L.mlp, DenseMlp):
                mlp = {"kind": "dense", "ff": L.mlp.ff}
            else:
                mlp = {"kind": "moe", "expert": {"ff": L.mlp.expert_ff},
                       "router": {"experts": L.mlp.experts, "top": L.mlp.top}}
                if L.mlp.shared_ff:
                    mlp["shared"] = {"ff": L.mlp.shared_ff}
            layers.append({"type": L.type, "mlp": mlp,
                           "mixer": {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}})
        d = {"architecture": "Sezazen", "vocab": self.vocab, "width": self.width, "max_positions": self.max_positions,
             "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale}, "layers": layers}
        if self.loop is not None:
            d["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        if self.eos_token_id is not None:
            d["eos_token_id"] = list(self.eos_token_id)
        return d

    # ------------------------------------------------------------------ the plan
    def run_order(self) -> list:
        """[(layer, pass number or None)]: the layers before the loop, the looped range `times` times, the rest."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        lp = self.loop
        return [(i, None) for i in range(lp.start)] + \
               [(i, t) for t in range(lp.times) for i in range(lp.start, lp.stop)] + \
               [(i, None) for i in range(lp.stop, n)]

    def plan(self) -> ModelPlan:
        c = self
        norm = PartSpec("rms_norm", {"size": c.width, "eps": c.norm_eps})
        blocks = []
        for L in c.layers:
            m = L.mixer
            # no rotation; every earlier key is visible; a sink of score zero in the softmax
            mixer = PartSpec("paged_attention", {
                "hidden_size": c.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                "value_dim": m.vdim, "position": PartSpec("no_position", {}), "window": ("full", 0),
                "softmax_scale": m.scale, "sink_logit": SINK_LOGIT})
            parts = {"mixer_norm": norm, "mixer": mixer}
            if isinstance(L.mlp, DenseMlp):
                parts.update(ffn_norm=norm, ffn=PartSpec("dense_swiglu", {"hidden_size": c.width, "intermediate_size": L.mlp.ff}))
            elif isinstance(L.mlp, MoeMlp):
                parts.update(ffn_norm=norm, ffn=PartSpec("moe_sigmoid_prescaled", {
                    "hidden_size": c.width, "num_experts": L.mlp.experts, "top_k": L.mlp.top,
                    "expert_size": L.mlp.expert_ff, "shared_size": L.mlp.shared_ff, "activation": "relu2"}))
            blocks.append(BlockSpec("prenorm_residual", parts))
        order = []
        for run, (i, t) in enumerate(c.run_order()):
            if t is not None and i == c.loop.start:
                order.append(JunctionCall(0, t))               # before every pass of the loop, the first too
            order.append(LayerCall(i, run, True))              # every run of a layer has a cache of its own
        junctions = ()
        if c.loop is not None:
            junctions = (PartSpec("reinject_linear", {"hidden_size": c.width, "steps": c.loop.times}),)
        return ModelPlan(hidden_size=c.width, vocab_size=c.vocab, blocks=tuple(blocks), order=tuple(order),
                         final_norm=norm, tie_word_embeddings=True, max_positions=c.max_positions,
                         embedding_scale=c.embedding_scale, position_table=c.max_positions,
                         junctions=junctions).validate()

    # ------------------------------------------------------------------ tensor names
    def weight_bindings(self) -> list:
        c = self
        d = c.width
        B = WeightBinding
        out = [B("embed.weight", "embed", (c.vocab, d)), B("positions.weight", "pos", (c.max_positions, d))]
        if c.loop is not None:
            out += [B("junctions.0.in_proj", "loop.in", (d, 2 * d)), B("junctions.0.step", "loop.step", (c.loop.times, d))]
        for i, L in enumerate(c.layers):
            s, t, m = f"l{i}.", f"layers.{i}.", L.mixer
            out += [B(t + "mixer_norm.weight", s + "norm1", (d,), init="ones"),
                    B(t + "mixer.q_proj", s + "mix.q", (m.heads * m.dim, d)),
                    B(t + "mixer.k_proj", s + "mix.k", (m.kv_heads * m.dim, d)),
                    B(t + "mixer.v_proj", s + "mix.v", (m.kv_heads * m.vdim, d)),
                    B(t + "mixer.o_proj", s + "mix.o", (d, m.heads * m.vdim))]
            if L.mlp is None:
                continue
            out.append(B(t + "ffn_norm.weight", s + "norm2", (d,), init="ones"))
            if isinstance(L.mlp, DenseMlp):
                f = L.mlp.ff
                out += [B(t + "ffn.gate_proj", s + "mlp.gate", (f, d)), B(t + "ffn.up_proj", s + "mlp.up", (f, d)),
                        B(t + "ffn.down_proj", s + "mlp.down", (d, f))]
            else:
                f, E = L.mlp.expert_ff, L.mlp.experts
                out += [B(t + "ffn.router", s + "mlp.router", (E, d)),
                        B(t + "ffn.experts_up", tuple(f"{s}mlp.e{e}.up" for e in range(E)), (f, d)),
                        B(t + "ffn.experts_down", tuple(f"{s}mlp.e{e}.down" for e in range(E)), (d, f))]
                if L.mlp.shared_ff:
                    fs = L.mlp.shared_ff
                    out += [B(t + "ffn.shared_up_proj", s + "mlp.shared.up", (fs, d)),
                            B(t + "ffn.shared_down_proj", s + "mlp.shared.down", (d, fs))]
        out.append(B("final_norm.weight", "final.norm", (d,), init="ones"))
        return out

    def unused_tensor_names(self) -> set:
        """What a file may carry for parts this configuration switches off: the second norm of a layer without a
        feed-forward, the loop's tensors of a model without a loop."""
        names = {f"l{i}.norm2" for i, L in enumerate(self.layers) if L.mlp is None}
        if self.loop is None:
            names |= {"loop.in", "loop.step"}
        return names

    checkpoint_prefixes = ("",)
    ignored_prefixes = ()
