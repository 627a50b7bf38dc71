"""Typed configuration of the Mibezen decoder, read from its config.json.

The file lists the layers one by one: `layers[i]` gives the layer's `type` (which mixer it has), the
mixer's sizes (`mixer`) and its feed-forward (`mlp`, or null for none).  Two mixers exist:

  latent_attention   queries, keys and values pass through low-rank latents; a part of every query head and
                     one key part shared by all heads rotate with the position (wavelengths stretched by the
                     YaRN rule when `rot.scaling` is given); every earlier position is visible; only the
                     latent and the shared key part are cached.
  attention          grouped-query attention without rotation: a bias slope_h * (i - j) is taken off the
                     scores, sight may be limited to the query's own chunk (`mask.size`), every head has a
                     learned sink in its softmax, and values may be blended with those of the first layer
                     that says `v_mix`.

Both gate every head's output with sigmoid(W_g h).  Feed-forwards: `dense` (down(relu(up h)^2)) or `moe`
(softmax router over all experts, the `top` largest renormalised, gated SiLU experts).  The norms store their
gains around zero; the output head is a tensor of its own and the logits are soft-capped.

Every size and every constant that the file gives is read from it; what the design fixes (the slopes'
formula, the amplitude 0.1 ln(factor) + 1 of the stretched rotation, the activations) is stated here and in `plan()`.

Tensor names: `embed`, `head`, `final.norm`, per layer `l<i>.norm1`, `l<i>.norm2`,
`l<i>.mix.{q,k,v,vmix,sink,g,o}` or `l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,g,o}`, and `l<i>.mlp.{up,down}`
or `l<i>.mlp.router`, `l<i>.mlp.e<j>.{gate,up,down}`; linear weights `[out, in]`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .registry import register_architecture
from .specs import BlockSpec, ConfigError, LayerCall, ModelPlan, PartSpec, WeightBinding

#: positions a request may reach when the file names no limit of its own
DEFAULT_MAX_POSITIONS = 1 << 20


def _need(d, key, where):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key `{where}{key}` is missing")
    return d[key]


def distance_slopes(heads: int) -> list:
    """slope_h = 2^(-8 (h + 1) / heads) for head h = 0 .. heads - 1."""
    return [2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)]


@dataclass(frozen=True)
class RotScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class LatentMixer:
    heads: int
    dim: int                  # unrotated query/key elements of a head
    rot_dim: int              # rotated ones
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_scaling: Optional[RotScaling]


@dataclass(frozen=True)
class ChunkMixer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int                # 0: every earlier position is visible
    v_mix: bool


@dataclass(frozen=True)
class DenseMlp:
    ff: int


@dataclass(frozen=True)
class MoeMlp:
    experts: int
    top: int
    expert_ff: int


@dataclass(frozen=True)
class MibezenLayer:
    type: str
    mixer: object             # LatentMixer | ChunkMixer
    mlp: object               # DenseMlp | MoeMlp | None


@register_architecture("Mibezen")
@dataclass(frozen=True)
class MibezenConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple
    logit_softcap: Optional[float] = None
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_id: Optional[tuple] = None

    MIXERS = ("latent_attention", "attention")

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict) -> "MibezenConfig":
        layers = []
        for i, L in enumerate(_need(raw, "layers", "")):
            at = f"layers[{i}]."
            kind = _need(L, "type", at)
            m, mat = _need(L, "mixer", at), at + "mixer."
            if kind == "latent_attention":
                rot = _need(m, "rot", mat)
                sc = rot.get("scaling")
                scaling = None
                if sc:
                    scaling = RotScaling(*(float(_need(sc, k, mat + "rot.scaling.")) for k in ("factor", "original", "fast", "slow")))
                rot_dim = int(_need(m, "rot_dim", mat))
                if int(rot.get("dims", rot_dim)) != rot_dim:
                    raise ConfigError(f"config.json: {mat}rot.dims {rot.get('dims')} differs from rot_dim {rot_dim}")
                mixer = LatentMixer(heads=int(_need(m, "heads", mat)), dim=int(_need(m, "dim", mat)), rot_dim=rot_dim,
                                    vdim=int(_need(m, "vdim", mat)), q_rank=int(_need(m, "q_rank", mat)),
                                    kv_rank=int(_need(m, "kv_rank", mat)), scale=float(_need(m, "scale", mat)),
                                    rot_base=float(_need(rot, "base", mat + "rot.")), rot_scaling=scaling)
            elif kind == "attention":
                heads = int(_need(m, "heads", mat))
                mask = m.get("mask")
                mixer = ChunkMixer(heads=heads, kv_heads=int(m.get("kv_heads") or heads), dim=int(_need(m, "dim", mat)),
                                   vdim=int(m.get("vdim") or m["dim"]), scale=float(_need(m, "scale", mat)),
                                   chunk=int(_need(mask, "size", mat + "mask.")) if mask else 0,
                                   v_mix=bool(m.get("v_mix")))
            else:
                raise ConfigError(f"config.json: {at}type {kind!r} is not a mixer of this design (known: {', '.join(cls.MIXERS)})")
            f = L.get("mlp")
            if f is None:
                mlp = None
            else:
                fk = _need(f, "kind", at + "mlp.")
                if fk == "dense":
                    mlp = DenseMlp(ff=int(_need(f, "ff", at + "mlp.")))
                elif fk == "moe":
                    r = _need(f, "router", at + "mlp.")
                    mlp = MoeMlp(experts=int(_need(r, "experts", at + "mlp.router.")), top=int(_need(r, "top", at + "mlp.router.")),
                                 expert_ff=int(_need(_need(f, "expert", at + "mlp."), "ff", at + "mlp.expert.")))
                else:
                    raise ConfigError(f"config.json: {at}mlp.kind {fk!r} is unknown (dense, moe)")
            layers.append(MibezenLayer(kind, mixer, mlp))
        eos = raw.get("eos_token_id")
        if isinstance(eos, int):
            eos = (eos,)
        elif eos is not None:
            eos = tuple(int(x) for x in eos)
        cap = raw.get("logit_softcap")
        cfg = cls(vocab=int(_need(raw, "vocab", "")), width=int(_need(raw, "width", "")),
                  norm_eps=float(_need(_need(raw, "norm", ""), "eps", "norm.")), layers=tuple(layers),
                  logit_softcap=float(cap) if cap else None,
                  max_positions=int(raw.get("max_positions") or DEFAULT_MAX_POSITIONS), eos_token_id=eos)
        cfg.validate()
        return cfg

    def validate(self):
        c = self
        for k, v in {"vocab": c.vocab, "width": c.width, "max_positions": c.max_positions}.items():
            if v <= 0:
                raise ConfigError(f"`{k}` must be positive, got {v}")
        if not c.norm_eps > 0:
            raise ConfigError("norm.eps must be positive")
        if c.logit_softcap is not None and not c.logit_softcap > 0:
            raise ConfigError("logit_softcap must be positive")
        if not c.layers:
            raise ConfigError("a model needs at least one layer")
        first_mix = None
        for i, L in enumerate(c.layers):
            m, at = L.mixer, f"layers[{i}].mixer"
            if isinstance(m, LatentMixer):
                if min(m.heads, m.dim, m.rot_dim, m.vdim, m.q_rank, m.kv_rank) < 1:
                    raise ConfigError(f"{at}: heads, dim, rot_dim, vdim, q_rank and kv_rank must be positive")
                if m.rot_dim % 2:
                    raise ConfigError(f"{at}: rot_dim {m.rot_dim} must be even (elements rotate in pairs)")
                if m.rot_base <= 1:
                    raise ConfigError(f"{at}.rot.base must exceed 1")
                s = m.rot_scaling
                if s is not None and (s.factor <= 0 or s.original <= 0 or s.fast <= 0 or s.slow <= 0):
                    raise ConfigError(f"{at}.rot.scaling: factor, original, fast and slow must be positive")
            else:
                if min(m.heads, m.kv_heads, m.dim, m.vdim) < 1 or m.chunk < 0:
                    raise ConfigError(f"{at}: heads, kv_heads, dim, vdim and mask.size must be positive")
                if m.heads % m.kv_heads:
                    raise ConfigError(f"{at}: {m.heads} heads are no multiple of {m.kv_heads} kv_heads")
                if m.v_mix:
                    if first_mix is None:
                        first_mix = (i, m)
                    elif (m.kv_heads, m.vdim) != (first_mix[1].kv_heads, first_mix[1].vdim):
                        raise ConfigError(f"{at}: v_mix needs the {first_mix[1].kv_heads} kv heads of {first_mix[1].vdim} "
                                          f"elements that layer {first_mix[0]} has")
            if isinstance(L.mlp, DenseMlp) and L.mlp.ff < 1:
                raise ConfigError(f"layers[{i}].mlp.ff must be positive")
            if isinstance(L.mlp, MoeMlp):
                f = L.mlp
                if f.experts < 1 or not 1 <= f.top <= f.experts:
                    raise ConfigError(f"layers[{i}].mlp.router: top {f.top} must lie in 1..experts ({f.experts})")
                if f.expert_ff < 1:
                    raise ConfigError(f"layers[{i}].mlp.expert.ff must be positive")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        layers = []
        for L in self.layers:
            m = L.mixer
            if isinstance(m, LatentMixer):
                rot = {"base": m.rot_base, "dims": m.rot_dim}
                if m.rot_scaling is not None:
                    s = m.rot_scaling
                    rot["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
                mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "q_rank": m.q_rank,
                         "kv_rank": m.kv_rank, "scale": m.scale, "rot": rot}
            else:
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                         "v_mix": m.v_mix}
                if m.chunk:
                    mixer["mask"] = {"size": m.chunk}
            if L.mlp is None:
                mlp = None
            elif isinstance(L.mlp, DenseMlp):
                mlp = {"kind": "dense", "ff": L.mlp.ff}
            else:
                mlp = {"kind": "moe", "expert": {"ff": L.mlp.expert_ff},
                       "router": {"experts": L.mlp.experts, "top": L.mlp.top}}
            layers.append({"type": L.type, "mixer": mixer, "mlp": mlp})
        d = {"architecture": "Mibezen", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "layers": layers}
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id is not None:
            d["eos_token_id"] = list(self.eos_token_id)
        return d

    # ------------------------------------------------------------------ the plan
    def first_mixing_layer(self):
        """Index of the first layer that says v_mix (its values are what the later ones blend in), or None."""
        for i, L in enumerate(self.layers):
            if isinstance(L.mixer, ChunkMixer) and L.mixer.v_mix:
                return i
        return None

    def plan(self) -> ModelPlan:
        c = self
        # the gains are stored as their distance from one
        norm = PartSpec("rms_norm", {"size": c.width, "eps": c.norm_eps, "gain_offset": 1.0})
        first_mix = c.first_mixing_layer()
        blocks = []
        for i, L in enumerate(c.layers):
            m = L.mixer
            if isinstance(m, LatentMixer):
                s = m.rot_scaling
                position = PartSpec("rotary_yarn", {
                    "rotary_dim": m.rot_dim, "theta": m.rot_base,
                    "scaling": None if s is None else {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}})
                mixer = PartSpec("latent_attention", {
                    "hidden_size": c.width, "num_heads": m.heads, "head_dim": m.dim, "rotary_dim": m.rot_dim,
                    "value_dim": m.vdim, "q_rank": m.q_rank, "kv_rank": m.kv_rank, "softmax_scale": m.scale,
                    "norm_eps": c.norm_eps, "position": position, "head_gate": True})
            else:
                value_mix = None
                if m.v_mix:
                    value_mix = "source" if i == first_mix else "blend"
                mixer = PartSpec("paged_attention", {
                    "hidden_size": c.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                    "value_dim": m.vdim, "position": PartSpec("no_position", {}),
                    "window": ("chunk", m.chunk) if m.chunk else ("full", 0), "softmax_scale": m.scale,
                    "head_sinks": True, "distance_slopes": tuple(distance_slopes(m.heads)),
                    "head_gate": True, "value_mix": value_mix})
            parts = {"mixer_norm": norm, "mixer": mixer}
            if isinstance(L.mlp, DenseMlp):
                parts.update(ffn_norm=norm, ffn=PartSpec("dense_activation", {
                    "hidden_size": c.width, "intermediate_size": L.mlp.ff, "activation": "relu2"}))
            elif isinstance(L.mlp, MoeMlp):
                parts.update(ffn_norm=norm, ffn=PartSpec("moe_softmax_topk", {
                    "hidden_size": c.width, "num_experts": L.mlp.experts, "top_k": L.mlp.top, "expert_size": L.mlp.expert_ff}))
            blocks.append(BlockSpec("prenorm_residual", parts))
        order = tuple(LayerCall(i, i, True) for i in range(len(c.layers)))
        return ModelPlan(hidden_size=c.width, vocab_size=c.vocab, blocks=tuple(blocks), order=order,
                         final_norm=norm, tie_word_embeddings=False, max_positions=c.max_positions,
                         logit_softcap=c.logit_softcap).validate()

    # ------------------------------------------------------------------ tensor names
    def weight_bindings(self) -> list:
        c = self
        d = c.width
        B = WeightBinding
        out = [B("embed.weight", "embed", (c.vocab, d))]
        for i, L in enumerate(c.layers):
            s, t, m = f"l{i}.", f"layers.{i}.", L.mixer
            out.append(B(t + "mixer_norm.weight", s + "norm1", (d,)))
            if isinstance(m, LatentMixer):
                out += [B(t + "mixer.q_down", s + "mix.dq", (m.q_rank, d)),
                        B(t + "mixer.q_latent_norm", s + "mix.dq.norm", (m.q_rank,), init="ones"),
                        B(t + "mixer.q_up", s + "mix.uq", (m.heads * (m.dim + m.rot_dim), m.q_rank)),
                        B(t + "mixer.kv_down", s + "mix.dkv", (m.kv_rank + m.rot_dim, d)),
                        B(t + "mixer.kv_latent_norm", s + "mix.dkv.norm", (m.kv_rank,), init="ones"),
                        B(t + "mixer.k_up", s + "mix.uk", (m.heads * m.dim, m.kv_rank)),
                        B(t + "mixer.v_up", s + "mix.uv", (m.heads * m.vdim, m.kv_rank)),
                        B(t + "mixer.gate_proj", s + "mix.g", (m.heads, d)),
                        B(t + "mixer.o_proj", s + "mix.o", (d, m.heads * m.vdim))]
            else:
                out += [B(t + "mixer.q_proj", s + "mix.q", (m.heads * m.dim, d)),
                        B(t + "mixer.k_proj", s + "mix.k", (m.kv_heads * m.dim, d)),
                        B(t + "mixer.v_proj", s + "mix.v", (m.kv_heads * m.vdim, d)),
                        B(t + "mixer.sinks", s + "mix.sink", (m.heads,)),
                        B(t + "mixer.gate_proj", s + "mix.g", (m.heads, d)),
                        B(t + "mixer.o_proj", s + "mix.o", (d, m.heads * m.vdim))]
                if m.v_mix:
                    out.append(B(t + "mixer.value_mix", s + "mix.vmix", ()))
            if L.mlp is None:
                continue
            out.append(B(t + "ffn_norm.weight", s + "norm2", (d,)))
            if isinstance(L.mlp, DenseMlp):
                f = L.mlp.ff
                out += [B(t + "ffn.up_proj", s + "mlp.up", (f, d)), B(t + "ffn.down_proj", s + "mlp.down", (d, f))]
            else:
                f, E = L.mlp.expert_ff, L.mlp.experts
                out += [B(t + "ffn.router", s + "mlp.router", (E, d)),
                        B(t + "ffn.experts_gate", tuple(f"{s}mlp.e{e}.gate" for e in range(E)), (f, d)),
                        B(t + "ffn.experts_up", tuple(f"{s}mlp.e{e}.up" for e in range(E)), (f, d)),
                        B(t + "ffn.experts_down", tuple(f"{s}mlp.e{e}.down" for e in range(E)), (d, f))]
        out += [B("final_norm.weight", "final.norm", (d,)), B("head.weight", "head", (c.vocab, d))]
        return out

    def unused_tensor_names(self) -> set:
        """What a file may carry for parts this configuration switches off: the second norm of a layer without a
        feed-forward, the blending weight of a layer that does not blend."""
        names = {f"l{i}.norm2" for i, L in enumerate(self.layers) if L.mlp is None}
        names |= {f"l{i}.mix.vmix" for i, L in enumerate(self.layers)
                  if isinstance(L.mixer, ChunkMixer) and not L.mixer.v_mix}
        return names

    checkpoint_prefixes = ("",)
    ignored_prefixes = ()
