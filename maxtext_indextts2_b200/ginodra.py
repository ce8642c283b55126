"""The Ginodra design: a decoder of parallel layers whose config.json lists them one by one.

A layer has ONE norm, and its mixer and feed-forward both read it:

    h = gnorm(x, norm1)                                  (RMS norm in `norm.groups` consecutive parts, times the weight)
    x += residual_mult * (mixer(h + conv_a(h)) + ff(h + conv_b(h)))

with conv a causal per-channel convolution over time (`canon.taps` taps; the last taps - 1 rows of h are state of a sequence)
and ff(z) = down(relu(up z)^2).  Mixers:

* ``attention``        -- grouped-query softmax attention without rotation: per-head RMS norm of queries and keys, a distance
                          penalty slope_h * (i - j) with slope_h = 2^(-8 (h + 1) / H), a sliding window, a sigmoid gate per head.
                          A layer with ``kv_from: j`` has no key / value projections and reads layer j's cache.
* ``latent_attention`` -- queries through a normed latent, keys and values expanded from a cached normed latent plus one rotated
                          key part shared by the heads (rotate-half pairing), a sink in the softmax's denominator, a gate per head.
* ``general_delta``    -- a matrix state per head that decays per key channel and from which, before a new key / value pair is
                          written, what it holds along the unit key is partly removed; per-head RMS norm, weight and sigmoid gate
                          on the read-out.

The logits are the (group-)normed stream times the embedding table, times `logit_scale`, soft-capped.

This module is the design's entry in the framework: config.json -> config keys (`config_keys`), checks (`validate_layer_specs`),
safetensors names -> layer descriptors of the layered engine (`model_plan`), random weights of any size (`random_tensors`).  No
arithmetic of the model happens here.  On the device every layer is a MTX_NORM_PARALLEL layer with one sub-mixer descriptor: the
softmax attention (with its optional norms, slopes, gate and shared pools), the latent attention, or the delta-rule recurrence.
"""

from __future__ import annotations

import math
from typing import Any, Dict, List, Optional

import torch

from .gugidra import TILE_ROWS, _need, _shape, rot_frequencies

MIXERS = ("attention", "latent_attention", "general_delta")
DELTA_DECAY_RATE = math.exp(-0.5)  # w = exp(-DELTA_DECAY_RATE * sigmoid(.))
DELTA_KEY_EPS = 1e-6               # u = k / sqrt(|k|^2 + DELTA_KEY_EPS)


def distance_slopes(heads: int) -> torch.Tensor:
  """slope_h = 2^(-8 (h + 1) / heads)."""
  return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=torch.float32)


def config_keys(model: dict) -> dict:
  """config.json of a Ginodra model -> keys of configs/base.yml."""
  layers = model["layers"]
  validate_layer_specs(layers)
  ffs = [int(l["mlp"]["ff"]) for l in layers if l.get("mlp")]
  first = layers[0]["mixer"]
  return dict(
      base_emb_dim=int(model["width"]),
      vocab_size=int(model["vocab"]),
      base_num_decoder_layers=len(layers),
      global_parameter_scale=1,
      normalization_layer_epsilon=float(model["norm"]["eps"]),
      norm_groups=int(model["norm"].get("groups", 1)),
      residual_multiplier=float(model.get("residual_mult", 1.0)),
      input_conv_taps=int(model["canon"]["taps"]) if model.get("canon") else 0,  # (0: the model has no input convolutions)
      logits_scale=float(model.get("logit_scale", 1.0)),
      final_logits_soft_cap=float(model.get("logit_softcap") or 0.0),
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
    if l["type"] == "attention":
      _need(m, ("heads", "kv_heads", "dim", "vdim", "scale"), where)
      if int(m["heads"]) % int(m["kv_heads"]):
        raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
      src = m.get("kv_from")
      if src is not None:
        src = int(src)
        if not 0 <= src < i or specs[src].get("type") != "attention" or specs[src]["mixer"].get("kv_from") is not None:
          raise ValueError(f"layer {i}: kv_from must name an earlier attention layer with projections of its own")
        o = specs[src]["mixer"]
        if any(int(o[k]) != int(m[k]) for k in ("kv_heads", "dim", "vdim")):
          raise ValueError(f"layer {i}: its key / value geometry differs from layer {src}'s, whose cache it reads")
    elif l["type"] == "latent_attention":
      _need(m, ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "rot", "scale"), where)
      if int(m["rot_dim"]) % 2 or int(m["rot"]["dims"]) != int(m["rot_dim"]):
        raise ValueError(f"layer {i}: rot_dim must be even and equal to rot.dims")
    else:
      _need(m, ("heads", "dim"), where)
    f = l.get("mlp")
    if f is not None:
      if f.get("kind", "dense") != "dense":
        raise ValueError(f"layer {i}: feed-forward kind {f.get('kind')!r}; this design has dense ones")
      _need(f, ("ff",), f"layer {i}: mlp")


def _conv_taps_major(t: Dict[str, torch.Tensor], name: str, E: int, taps: int) -> torch.Tensor:
  """[width, taps] as stored -> [taps, width] fp32 (the kernels read a tap's weights of neighbouring channels together).  A model
  without input convolutions (taps == 0) gets one tap of zeros: h + 0 * h."""
  if taps == 0:
    return torch.zeros(1, E, dtype=torch.float32, device=t["embed"].device)
  return _shape(t[name].to(torch.float32), (E, taps), name).t().contiguous()


def layer_plan(config, tensors: Dict[str, torch.Tensor], i: int) -> Dict[str, Any]:
  """What layer i hands to the layered engine: sizes and scalars (python numbers) and host tensors; matrices keep their stored
  dtype.  All projections of the mixer's input are concatenated into one matrix in the order the device reads them, and the
  mixer's output projection is concatenated with the feed-forward's down-projection along their inputs."""
  spec = config.layer_specs[i]
  E, taps = int(config.emb_dim), int(config.input_conv_taps)
  t, p = tensors, f"l{i}.mix."
  dev = tensors["embed"].device
  f32 = lambda name: t[name].to(torch.float32)
  m = spec["mixer"]
  plan: Dict[str, Any] = dict(mixer="composite", norm_style="parallel", attn=None, rec=None, latent=None, moe=None, ff_kind="relu2", ff=0,
                              residual_mult=float(config.residual_multiplier), conv_taps=max(taps, 1),
                              norm1=_shape(f32(f"l{i}.norm1"), (E,), f"l{i}.norm1"), conv1=_conv_taps_major(t, f"l{i}.canon1", E, taps), conv2=None)
  rows: List[torch.Tensor] = []
  if spec["type"] == "attention":
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    src = m.get("kv_from")
    rows.append(_shape(t[p + "q"], (H * d, E), p + "q"))
    if src is None:
      rows += [_shape(t[p + "k"], (G * d, E), p + "k"), _shape(t[p + "v"], (G * dv, E), p + "v")]
    rows.append(_shape(t[p + "g"], (H, E), p + "g"))
    window = int(m["mask"]["size"]) if m.get("mask") else 0
    plan["attn"] = dict(heads=H, kv_heads=G, dim=d, vdim=dv, window=window, rot_dims=0, values_are_keys=0, scale=float(m["scale"]), out_scale=1.0,
                        rot_freq=None, rot_half=0, shared_kv=0 if src is None else 1, kv_from=None if src is None else int(src), head_gate=1,
                        q_norm=_shape(f32(p + "q.norm"), (d,), p + "q.norm"),
                        k_norm=_shape(f32(p + "k.norm"), (d,), p + "k.norm") if src is None else None,
                        slopes=distance_slopes(H), sink=None)
    k_mix = H * dv
  elif spec["type"] == "latent_attention":
    H, d, dr, dv = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"])
    qr, kr = int(m["q_rank"]), int(m["kv_rank"])
    rows += [_shape(t[p + "dq"], (qr, E), p + "dq"), _shape(t[p + "dkv"], (kr + dr, E), p + "dkv"), _shape(t[p + "g"], (H, E), p + "g")]
    uk = _shape(t[p + "uk"], (H * d, kr), p + "uk")
    plan["latent"] = dict(heads=H, dim=d, rot_dim=dr, vdim=dv, q_rank=qr, kv_rank=kr, rot_half=1, scale=float(m["scale"]),
                          rot_freq=rot_frequencies(dr, float(m["rot"]["base"])) if dr else None,
                          q_norm=_shape(f32(p + "dq.norm"), (qr,), p + "dq.norm"), kv_norm=_shape(f32(p + "dkv.norm"), (kr,), p + "dkv.norm"),
                          sink=_shape(f32(p + "sink"), (H,), p + "sink") if (p + "sink") in t else None,
                          w_uq=_shape(t[p + "uq"], (H * (d + dr), qr), p + "uq"),
                          w_uk_t=uk.reshape(H, d, kr).transpose(1, 2).contiguous(),  # [H, kv_rank, dim]
                          w_uv=_shape(t[p + "uv"], (H * dv, kr), p + "uv").reshape(H, dv, kr).contiguous())
    k_mix = H * dv
  else:
    H, d = int(m["heads"]), int(m["dim"])
    for name in ("r", "k", "v", "g", "a"):
      rows.append(_shape(t[p + name], (H * d, E), p + name))
    rank = int(t[p + "w1"].shape[0])
    rows.append(_shape(t[p + "w1"], (rank, E), p + "w1"))
    plan["rec"] = dict(kind="delta", heads=H, dim=d, vdim=d, decay_rank=rank, gate_silu=0, q_scale=1.0, tau=1.0, gate_cap=0.0, denom_eps=0.0,
                       out_scale=1.0, decay_rate=DELTA_DECAY_RATE, key_eps=DELTA_KEY_EPS,
                       decay_up_t=_shape(f32(p + "w2"), (H * d, rank), p + "w2").t().contiguous(),
                       decay_bias=_shape(f32(p + "w0"), (H * d,), p + "w0"),
                       gate_bias=_shape(f32(p + "a.b"), (H * d,), p + "a.b"),
                       out_norm=_shape(f32(p + "norm"), (H * d,), p + "norm"))
    k_mix = H * d
  w_in = torch.cat(rows, dim=0)
  pad = (-w_in.shape[0]) % TILE_ROWS
  if pad and E % 64 == 0:
    w_in = torch.cat([w_in, torch.zeros(pad, E, dtype=w_in.dtype, device=dev)], dim=0)
  wo = [_shape(t[p + "o"], (E, k_mix), p + "o")]
  f = spec.get("mlp")
  if f is not None:
    F = int(f["ff"])
    q = f"l{i}.mlp."
    plan.update(ff=F, w_gate_up=_shape(t[q + "up"], (F, E), q + "up"), conv2=_conv_taps_major(t, f"l{i}.canon2", E, taps))
    wo.append(_shape(t[q + "down"], (E, F), q + "down"))
  plan.update(w_in=w_in, n_in=int(w_in.shape[0]), wo=torch.cat(wo, dim=1).contiguous())
  return plan


def model_plan(config, tensors: Dict[str, torch.Tensor]) -> Dict[str, Any]:
  E = int(config.emb_dim)
  layers = [layer_plan(config, tensors, i) for i in range(len(config.layer_specs))]
  return dict(
      embedding=tensors["embed"], head=tensors["embed"], final_gain=1.0, final_norm=_shape(tensors["final.norm"].to(torch.float32), (E,), "final.norm"),
      embed_scale=1.0, logit_softcap=float(config.final_logits_soft_cap or 0.0), logit_scale=float(config.logits_scale),
      norm_groups=int(config.norm_groups), layers=layers,
  )


def random_tensors(config, seed: int = 0, device: Any = "cpu") -> Dict[str, torch.Tensor]:
  """Random bf16 weights with the design's tensor names, for `config` (tests, benchmarks and smoke runs; made on `device`)."""
  g = torch.Generator(device=device).manual_seed(seed)
  E, V, taps = int(config.emb_dim), int(config.vocab_size), int(config.input_conv_taps)
  bf = torch.bfloat16

  def rn(*shape, std=1.0, mean=0.0):
    return (torch.randn(tuple(shape), generator=g, device=device) * std + mean).to(bf)

  lin = lambda n, k: rn(n, k, std=1.0 / math.sqrt(k))
  t = {"embed": rn(V, E), "final.norm": rn(E, std=0.1, mean=1.0)}
  for i, l in enumerate(config.layer_specs):
    p, m = f"l{i}.", l["mixer"]
    t[p + "norm1"] = rn(E, std=0.1, mean=1.0)
    if taps:
      t[p + "canon1"] = rn(E, taps, std=0.3)
    q = p + "mix."
    if l["type"] == "attention":
      H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
      t[q + "q"], t[q + "q.norm"], t[q + "g"], t[q + "o"] = lin(H * d, E), rn(d, std=0.1, mean=1.0), lin(H, E), lin(E, H * dv)
      if m.get("kv_from") is None:
        t[q + "k"], t[q + "v"], t[q + "k.norm"] = lin(G * d, E), lin(G * dv, E), rn(d, std=0.1, mean=1.0)
    elif l["type"] == "latent_attention":
      H, d, dr, dv, qr, kr = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"))
      t[q + "dq"], t[q + "dq.norm"], t[q + "uq"] = lin(qr, E), rn(qr, std=0.1, mean=1.0), lin(H * (d + dr), qr)
      t[q + "dkv"], t[q + "dkv.norm"] = lin(kr + dr, E), rn(kr, std=0.1, mean=1.0)
      t[q + "uk"], t[q + "uv"], t[q + "sink"] = lin(H * d, kr), lin(H * dv, kr), rn(H, std=1.0)
      t[q + "g"], t[q + "o"] = lin(H, E), lin(E, H * dv)
    else:
      H, d = int(m["heads"]), int(m["dim"])
      rank = int(m.get("rank", 16))
      for n in ("r", "k", "v", "g", "a"):
        t[q + n] = lin(H * d, E)
      t[q + "a.b"], t[q + "w1"], t[q + "w2"], t[q + "w0"] = rn(H * d, std=0.5), lin(rank, E), rn(H * d, rank, std=0.5), rn(H * d, std=1.0)
      t[q + "norm"], t[q + "o"] = rn(H * d, std=0.1, mean=1.0), lin(E, H * d)
    f = l.get("mlp")
    if f:
      F = int(f["ff"])
      t[p + "mlp.up"], t[p + "mlp.down"] = lin(F, E), lin(E, F)
      if taps:
        t[p + "canon2"] = rn(E, taps, std=0.3)
  return t


# -- config.json-shaped dicts (tests, benchmarks) ----------------------------------------------------------------------------


def model_dict(width: int, vocab: int, layers: List[dict], eps: float = 1e-5, groups: int = 1, taps: int = 4, residual_mult: float = 0.5,
               logit_scale: float = 1.0, logit_softcap: float = 30.0) -> dict:
  return {"architecture": "Ginodra", "width": width, "vocab": vocab, "norm": {"eps": eps, "groups": groups}, "canon": {"taps": taps},
          "residual_mult": residual_mult, "logit_scale": logit_scale, "logit_softcap": logit_softcap, "layers": layers}


def dense_ff(ff: int) -> dict:
  return {"kind": "dense", "ff": ff}


def attention_layer(heads: int, kv_heads: int, dim: int, vdim: Optional[int] = None, window: int = 0, scale: float = 0.0, kv_from: Optional[int] = None,
                    mlp: Optional[dict] = None) -> dict:
  m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim if vdim is None else vdim, "scale": scale or dim**-0.5}
  if window:
    m["mask"] = {"size": window}
  if kv_from is not None:
    m["kv_from"] = kv_from
  return {"type": "attention", "mixer": m, "mlp": mlp}


def latent_layer(heads: int, dim: int, rot_dim: int, vdim: int, q_rank: int, kv_rank: int, rot_base: float = 10000.0, scale: float = 0.0,
                 mlp: Optional[dict] = None) -> dict:
  return {"type": "latent_attention",
          "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                    "rot": {"base": rot_base, "dims": rot_dim}, "scale": scale or (dim + rot_dim) ** -0.5},
          "mlp": mlp}


def delta_layer(heads: int, dim: int, mlp: Optional[dict] = None, rank: int = 16) -> dict:
  return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "rank": rank}, "mlp": mlp}
