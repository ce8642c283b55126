"""The Ligidra design: a pre-norm decoder whose config.json lists its layers one by one.

The embedding row is RMS-normed (``embed.norm``).  A layer is

    h = rms(x) * norm1;   x += mixer(h + (h_prev - h) * shift)     (h_prev: the previous token's h, zero before the first)
    x += ff(rms(x) * norm2)                                        (a routed feed-forward, or none)
    x += unit(side.proj(gelu_tanh(side.gate x) * e)) * side.norm   (e: the layer's part of the token's row of ``side.embed``)

with rms(x) = x / sqrt(mean(x^2) + eps) = unit(x).  Mixers:

* ``attention``      -- grouped-query softmax attention: RMS norm of the WHOLE query / key projection (one weight per channel of
                        all heads), rotary positions on interleaved pairs with long wavelengths slowed down, a capped score
                        ``cap * tanh(s / cap)``, a sliding window plus ONE mean key / value per block of ``mask.pool`` tokens that lies
                        wholly before the window, a sink in the denominator.  ``kv_from: j`` reads layer j's cache.
* ``delta``          -- gated delta rule: q, k, v pass a short causal convolution and silu; unit q and k; per head a scalar decay
                        ``exp(-exp(A_log) softplus(a h + dt_bias))`` and a write strength ``sigmoid(b h)``; the state is decayed, the
                        value the decayed state already holds along k is taken off the written value; read-out RMS norm, silu gate.
* ``channel_delta``  -- the same with a decay per key channel from a low-rank projection, and a low-rank sigmoid gate.

Feed-forward: softmax router over all experts, the `top` largest scores as weights (not renormalised), silu-gated experts, a shared
expert.  The logits are the normed stream times the embedding table.

This module is the design's entry in the framework: config.json -> config keys (`config_keys`), checks (`validate_layer_specs`),
safetensors names -> layer descriptors of the layered engine (`model_plan`), random weights of any size (`random_tensors`).  No
arithmetic of the model happens here.  On the device every layer is a MTX_NORM_PRE layer: the token shift is a two-tap input
convolution over the sequence's ring of normed rows, the mixer a softmax attention (with its pooled pools) or a MTX_REC_GDELTA
recurrence, the feed-forward a MTX_FF_MOE with softmax scores.
"""

from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from .gugidra import TILE_ROWS, _interleave, _need, _shape

MIXERS = ("attention", "delta", "channel_delta")
UNIT_EPS = 1e-6  # inside the root of the recurrences' unit vectors


def scaled_rot_frequencies(dims: int, base: float, scaling: Optional[dict]) -> torch.Tensor:
  """Radians per position of the channel pair i < dims / 2, float64.  base^(-2i / dims); with `scaling` {factor, low, high,
  original}: a pair whose wavelength exceeds original / low turns `factor` times slower, one below original / high as it is, and
  between the two the frequency is blended linearly in original / wavelength."""
  f = float(base) ** (-2.0 * np.arange(dims // 2, dtype=np.float64) / dims)
  if scaling:
    factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
    wl = 2.0 * math.pi / f
    blend = (orig / wl - low) / (high - low) if high != low else np.ones_like(f)
    mid = (1.0 - blend) * f / factor + blend * f
    f = np.where(wl < orig / high, f, np.where(wl > orig / low, f / factor, mid))
  return torch.from_numpy(np.ascontiguousarray(f))


def config_keys(model: dict) -> dict:
  """config.json of a Ligidra model -> keys of configs/base.yml."""
  layers = model["layers"]
  validate_layer_specs(layers)
  ffs = [int(l["mlp"]["expert"]["ff"]) for l in layers if l.get("mlp")]
  first = layers[0]["mixer"]
  side = model.get("token_side") or {}
  return dict(
      base_emb_dim=int(model["width"]),
      vocab_size=int(model["vocab"]),
      base_num_decoder_layers=len(layers),
      global_parameter_scale=1,
      normalization_layer_epsilon=float(model["norm"]["eps"]),
      token_side_dim=int(side.get("dim") or 0),
      layer_specs=layers,
      # (the homogeneous keys describe the first layer; the engine reads layer_specs)
      base_num_query_heads=int(first["heads"]),
      base_num_kv_heads=int(first.get("kv_heads", first["heads"])),
      head_dim=int(first["dim"]),
      base_mlp_dim=max(ffs) if ffs else 0,
  )


def validate_layer_specs(specs: List[dict]) -> None:
  for i, l in enumerate(specs):
    if l.get("type") not in MIXERS:
      raise ValueError(f"layer {i}: mixer type {l.get('type')!r}; this design has {MIXERS}")
    m = l["mixer"]
    where = f"layer {i}: mixer"
    _need(m, ("heads", "kv_heads", "dim", "vdim"), where)
    if int(m["heads"]) % int(m["kv_heads"]):
      raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
    if l["type"] == "attention":
      _need(m, ("scale",), where)
      rot = m.get("rot")
      if rot and (int(rot["dims"]) % 2 or int(rot["dims"]) > int(m["dim"])):
        raise ValueError(f"layer {i}: rot.dims must be even and at most dim")
      mask = m.get("mask") or {}
      if int(mask.get("pool") or 0) and not int(mask.get("size") or 0):
        raise ValueError(f"layer {i}: pooled blocks need a window")
      src = m.get("kv_from")
      if src is not None:
        src = int(src)
        if not 0 <= src < i or specs[src].get("type") != "attention" or specs[src]["mixer"].get("kv_from") is not None:
          raise ValueError(f"layer {i}: kv_from must name an earlier attention layer with projections of its own")
        o = specs[src]["mixer"]
        if any(int(o[k]) != int(m[k]) for k in ("kv_heads", "dim", "vdim")):
          raise ValueError(f"layer {i}: its key / value geometry differs from layer {src}'s, whose cache it reads")
    else:
      _need(m, ("conv",), where)
      if int(m["conv"]) < 1:
        raise ValueError(f"layer {i}: the short convolution has at least one tap")
    f = l.get("mlp")
    if f is not None:
      if f.get("kind", "moe") != "moe":
        raise ValueError(f"layer {i}: feed-forward kind {f.get('kind')!r}; this design has routed ones")
      _need(f, ("expert", "router"), f"layer {i}: mlp")
      n, top = int(f["router"]["experts"]), int(f["router"]["top"])
      if not 1 <= top <= n:
        raise ValueError(f"layer {i}: top {top} of {n} experts")


def _taps_major(w: torch.Tensor) -> torch.Tensor:
  """[channels, taps] as stored -> [taps, channels] fp32 (a tap's weights of neighbouring channels lie together)."""
  return w.to(torch.float32).t().contiguous()


def layer_plan(config, tensors: Dict[str, torch.Tensor], i: int) -> Dict[str, Any]:
  """What layer i hands to the layered engine: sizes and scalars (python numbers) and host tensors; matrices keep their stored
  dtype.  All projections of the mixer's input are one matrix in the order the device reads them."""
  spec = config.layer_specs[i]
  E, eps = int(config.emb_dim), float(config.normalization_layer_epsilon)
  t, p = tensors, f"l{i}.mix."
  dev = tensors["embed"].device
  f32 = lambda name: t[name].to(torch.float32)
  m = spec["mixer"]
  shift = _shape(f32(f"l{i}.shift"), (E,), f"l{i}.shift")
  plan: Dict[str, Any] = dict(mixer="composite", norm_style="pre", attn=None, rec=None, latent=None, moe=None, ff_kind="moe", ff=0,
                              residual_mult=1.0, conv_taps=2, conv2=None,
                              norm1=_shape(f32(f"l{i}.norm1"), (E,), f"l{i}.norm1"),
                              # h + (h_prev - h) * shift = h + [shift * h_prev + (-shift) * h]: a two-tap convolution added to its input
                              conv1=torch.stack([shift, -shift]).contiguous())
  H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
  rows: List[torch.Tensor] = []
  if spec["type"] == "attention":
    src = m.get("kv_from")
    rows.append(_shape(t[p + "q"], (H * d, E), p + "q"))
    if src is None:
      rows += [_shape(t[p + "k"], (G * d, E), p + "k"), _shape(t[p + "v"], (G * dv, E), p + "v")]
    mask, rot = m.get("mask") or {}, m.get("rot")
    rd = int(rot["dims"]) if rot else 0
    plan["attn"] = dict(heads=H, kv_heads=G, dim=d, vdim=dv, window=int(mask.get("size") or 0), pool=int(mask.get("pool") or 0), rot_dims=rd,
                        values_are_keys=0, scale=float(m["scale"]), out_scale=1.0, softcap=float(m.get("softcap") or 0.0),
                        rot_freq=scaled_rot_frequencies(rd, float(rot["base"]), rot.get("scaling")) if rd else None, rot_half=0,
                        shared_kv=0 if src is None else 1, kv_from=None if src is None else int(src), head_gate=0, norm_whole=1,
                        q_norm=_shape(f32(p + "q.norm"), (H * d,), p + "q.norm"),
                        k_norm=_shape(f32(p + "k.norm"), (G * d,), p + "k.norm") if src is None else None,
                        slopes=None, sink=_shape(f32(p + "sink"), (H,), p + "sink") if (p + "sink") in t else None)
  else:
    taps = int(m["conv"])
    per_channel = spec["type"] == "channel_delta"
    rows += [_shape(t[p + "q"], (G * d, E), p + "q"), _shape(t[p + "k"], (G * d, E), p + "k"), _shape(t[p + "v"], (H * dv, E), p + "v"),
             _shape(t[p + "b"], (H, E), p + "b")]
    conv = torch.cat([_shape(t[p + "q.conv"], (G * d, taps), p + "q.conv"), _shape(t[p + "k.conv"], (G * d, taps), p + "k.conv"),
                      _shape(t[p + "v.conv"], (H * dv, taps), p + "v.conv")], dim=0)
    rec = dict(kind="gdelta", heads=H, kv_heads=G, dim=d, vdim=dv, decay_rank=0, gate_rank=0, gate_silu=1, q_scale=d**-0.5, tau=1.0, gate_cap=0.0,
               denom_eps=0.0, out_scale=1.0, key_eps=UNIT_EPS, conv_taps=taps, conv_w=_taps_major(conv),
               a_log=_shape(f32(p + "A_log"), (H,), p + "A_log"), out_norm=_shape(f32(p + "norm"), (dv,), p + "norm").repeat(H),
               decay_up2=None, w_gate_up=None)
    if per_channel:
      ra, rg = int(t[p + "a1"].shape[0]), int(t[p + "g1"].shape[0])
      rows += [_shape(t[p + "a1"], (ra, E), p + "a1"), _shape(t[p + "g1"], (rg, E), p + "g1")]
      a2 = _shape(t[p + "a2"], (H * d, ra), p + "a2")
      # (the up-projection twice along its inputs: the device feeds it the fp32 input split into two parts of the matmul dtype)
      rec.update(decay_rank=ra, gate_rank=rg, gate_silu=0, decay_up2=torch.cat([a2, a2], dim=1).contiguous(),
                 decay_bias=_shape(f32(p + "dt_bias"), (H * d,), p + "dt_bias"), w_gate_up=_shape(t[p + "g2"], (H * dv, rg), p + "g2"))
    else:
      rows += [_shape(t[p + "a"], (H, E), p + "a"), _shape(t[p + "g"], (H * dv, E), p + "g")]
      rec.update(decay_bias=_shape(f32(p + "dt_bias"), (H,), p + "dt_bias"))
    plan["rec"] = rec
  w_in = torch.cat(rows, dim=0)
  pad = (-w_in.shape[0]) % TILE_ROWS
  if pad and E % 64 == 0:
    w_in = torch.cat([w_in, torch.zeros(pad, E, dtype=w_in.dtype, device=dev)], dim=0)
  plan.update(w_in=w_in, n_in=int(w_in.shape[0]), wo=_shape(t[p + "o"], (E, H * dv), p + "o"))
  f = spec.get("mlp")
  if f is not None:
    q = f"l{i}.mlp."
    plan["norm2"] = _shape(f32(f"l{i}.norm2"), (E,), f"l{i}.norm2")

    def gated(prefix: str, F: int):
      return (_interleave(_shape(t[prefix + "gate"], (F, E), prefix + "gate"), _shape(t[prefix + "up"], (F, E), prefix + "up")),
              _shape(t[prefix + "down"], (E, F), prefix + "down"))

    n_exp, F, sh = int(f["router"]["experts"]), int(f["expert"]["ff"]), f.get("shared")
    parts = [gated(f"{q}e{e}.", F) for e in range(n_exp)]
    moe = dict(experts=n_exp, top=int(f["router"]["top"]), groups=1, keep_groups=1, ff=F, limit=0.0, shared_ff=0, shared_limit=0.0,
               score_softmax=1, plain_weights=1, act_silu=1, w_router=_shape(t[q + "router"], (n_exp, E), q + "router"), correction=None,
               w_gate_up=torch.stack([g for g, _ in parts]), w_down=torch.stack([d_ for _, d_ in parts]), shared_gate_up=None, shared_down=None)
    if sh:
      gu, dn = gated(q + "shared.", int(sh["ff"]))
      moe.update(shared_ff=int(sh["ff"]), shared_gate_up=gu, shared_down=dn)
    plan["moe"] = moe
  sd = int(config.token_side_dim)
  if sd:
    s = f"l{i}.side."
    gate = _shape(t[s + "gate"], (sd, E), s + "gate")
    pad = (-sd) % TILE_ROWS
    if pad and E % 64 == 0:  # zero rows up to a whole tile of the tensor-core GEMM
      gate = torch.cat([gate, torch.zeros(pad, E, dtype=gate.dtype, device=dev)], dim=0)
    plan["side"] = dict(dim=sd, col=i * sd, gate=gate, proj=_shape(t[s + "proj"], (E, sd), s + "proj"),
                        norm=_shape(f32(s + "norm"), (E,), s + "norm"))
  return plan


def model_plan(config, tensors: Dict[str, torch.Tensor]) -> Dict[str, Any]:
  E, V, n = int(config.emb_dim), int(config.vocab_size), len(config.layer_specs)
  layers = [layer_plan(config, tensors, i) for i in range(n)]
  sd = int(config.token_side_dim)
  return dict(
      embedding=_shape(tensors["embed"], (V, E), "embed"), head=tensors["embed"], final_gain=1.0,
      final_norm=_shape(tensors["final.norm"].to(torch.float32), (E,), "final.norm"),
      embed_norm=_shape(tensors["embed.norm"].to(torch.float32), (E,), "embed.norm"),
      side_embed=_shape(tensors["side.embed"], (V, n * sd), "side.embed") if sd else None,
      embed_scale=1.0, logit_softcap=0.0, logit_scale=1.0, norm_groups=1, layers=layers,
  )


def random_tensors(config, seed: int = 0, device: Any = "cpu") -> Dict[str, torch.Tensor]:
  """Random bf16 weights with the design's tensor names, for `config` (tests, benchmarks and smoke runs; made on `device`)."""
  g = torch.Generator(device=device).manual_seed(seed)
  E, V, sd, n = int(config.emb_dim), int(config.vocab_size), int(config.token_side_dim), len(config.layer_specs)
  bf = torch.bfloat16

  def rn(*shape, std=1.0, mean=0.0):
    return (torch.randn(tuple(shape), generator=g, device=device) * std + mean).to(bf)

  def un(*shape, lo=0.0, hi=1.0):
    return (torch.rand(tuple(shape), generator=g, device=device) * (hi - lo) + lo).to(bf)

  lin = lambda n_, k: rn(n_, k, std=1.0 / math.sqrt(k))
  t = {"embed": rn(V, E), "embed.norm": rn(E, std=0.1, mean=1.0), "final.norm": rn(E, std=0.1, mean=1.0)}
  if sd:
    t["side.embed"] = rn(V, n * sd)
  for i, l in enumerate(config.layer_specs):
    p, m = f"l{i}.", l["mixer"]
    t[p + "norm1"], t[p + "shift"] = rn(E, std=0.1, mean=1.0), un(E)
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = p + "mix."
    if l["type"] == "attention":
      t[q + "q"], t[q + "q.norm"], t[q + "sink"], t[q + "o"] = lin(H * d, E), rn(H * d, std=0.1, mean=1.0), rn(H, std=1.0), lin(E, H * dv)
      if m.get("kv_from") is None:
        t[q + "k"], t[q + "v"], t[q + "k.norm"] = lin(G * d, E), lin(G * dv, E), rn(G * d, std=0.1, mean=1.0)
    else:
      taps = int(m["conv"])
      t[q + "q"], t[q + "k"], t[q + "v"], t[q + "b"] = lin(G * d, E), lin(G * d, E), lin(H * dv, E), lin(H, E)
      t[q + "q.conv"], t[q + "k.conv"], t[q + "v.conv"] = rn(G * d, taps, std=0.5), rn(G * d, taps, std=0.5), rn(H * dv, taps, std=0.5)
      t[q + "A_log"], t[q + "norm"], t[q + "o"] = un(H, lo=-3.0, hi=0.5), rn(dv, std=0.1, mean=1.0), lin(E, H * dv)
      if l["type"] == "channel_delta":
        rank = int(m.get("rank", 8))
        t[q + "a1"], t[q + "a2"], t[q + "dt_bias"] = lin(rank, E), rn(H * d, rank, std=0.5), rn(H * d, std=1.0)
        t[q + "g1"], t[q + "g2"] = lin(rank, E), rn(H * dv, rank, std=0.5)
      else:
        t[q + "a"], t[q + "dt_bias"], t[q + "g"] = lin(H, E), rn(H, std=1.0), lin(H * dv, E)
    f = l.get("mlp")
    if f:
      t[p + "norm2"] = rn(E, std=0.1, mean=1.0)
      q = p + "mlp."

      def gated(prefix, F):
        t[prefix + "gate"], t[prefix + "up"], t[prefix + "down"] = lin(F, E), lin(F, E), lin(E, F)

      n_exp = int(f["router"]["experts"])
      for e in range(n_exp):
        gated(f"{q}e{e}.", int(f["expert"]["ff"]))
      t[q + "router"] = rn(n_exp, E, std=2.0 / math.sqrt(E))
      if f.get("shared"):
        gated(q + "shared.", int(f["shared"]["ff"]))
    if sd:
      t[p + "side.gate"], t[p + "side.proj"], t[p + "side.norm"] = lin(sd, E), lin(E, sd), rn(E, std=0.05, mean=0.3)
  return t


# -- config.json-shaped dicts (tests, benchmarks) ----------------------------------------------------------------------------


def model_dict(width: int, vocab: int, layers: List[dict], eps: float = 1e-6, side_dim: int = 0) -> dict:
  out = {"architecture": "Ligidra", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}
  if side_dim:
    out["token_side"] = {"dim": side_dim}
  return out


def moe_ff(experts: int, top: int, ff: int, shared_ff: int = 0) -> dict:
  out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
  if shared_ff:
    out["shared"] = {"ff": shared_ff}
  return out


def attention_layer(heads: int, kv_heads: int, dim: int, vdim: Optional[int] = None, window: int = 0, pool: int = 0, scale: float = 0.0,
                    softcap: float = 0.0, rot_dims: Optional[int] = None, rot_base: float = 10000.0, rot_scaling: Optional[dict] = None,
                    kv_from: Optional[int] = None, mlp: Optional[dict] = None) -> dict:
  m: Dict[str, Any] = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim if vdim is None else vdim, "scale": scale or dim**-0.5}
  if softcap:
    m["softcap"] = softcap
  rd = dim if rot_dims is None else rot_dims
  if rd:
    m["rot"] = {"base": rot_base, "dims": rd}
    if rot_scaling:
      m["rot"]["scaling"] = rot_scaling
  if window:
    m["mask"] = {"size": window}
    if pool:
      m["mask"]["pool"] = pool
  if kv_from is not None:
    m["kv_from"] = kv_from
  return {"type": "attention", "mixer": m, "mlp": mlp}


def delta_layer(heads: int, kv_heads: int, dim: int, vdim: int, taps: int = 4, per_channel: bool = False, rank: int = 8, mlp: Optional[dict] = None) -> dict:
  m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": taps}
  if per_channel:
    m["rank"] = rank  # (random_tensors reads it; a stored model gives the rank by its tensors' shapes)
  return {"type": "channel_delta" if per_channel else "delta", "mixer": m, "mlp": mlp}
