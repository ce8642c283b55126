"""A plain float64 restatement of the Ginodra design, one function per mechanism, for the tests.

Nothing here is shared with the engine: numpy only, whole sequences, O(n^2) attention written as loops over query positions, the
recurrence as the token loop that defines it.  `tensors` maps the stored names to float64 arrays, `model` is the config.json
dict.  Notation: E width, T tokens of one sequence, H heads, d per-head key size, dv per-head value size.

A layer with h = gnorm(x):  x <- x + m * (mixer(h + conv_a(h)) + ff(h + conv_b(h))).
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np


def sigmoid(z):
  return 1.0 / (1.0 + np.exp(-z))


def rms_unit(x, eps):
  """x / sqrt(mean(x^2) + eps) over the last axis."""
  return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def group_norm(x, w, groups: int, eps: float):
  """The last axis in `groups` equal consecutive parts, each brought to unit RMS on its own; then the weight."""
  shape = x.shape
  parts = x.reshape(shape[:-1] + (groups, shape[-1] // groups))
  return rms_unit(parts, eps).reshape(shape) * w


def causal_conv(h, w):
  """h [T, E], w [E, taps]: out[t] = sum_j w[:, j] * h[t - (taps - 1) + j], rows before the sequence count as zero."""
  T, E = h.shape
  taps = w.shape[1]
  padded = np.concatenate([np.zeros((taps - 1, E)), h], axis=0)
  out = np.zeros_like(h)
  for j in range(taps):
    out += padded[j : j + T] * w[:, j]
  return out


def squared_relu_ff(h, up, down):
  a = np.maximum(h @ up.T, 0.0)
  return (a * a) @ down.T


def rotate_half(x, positions, base: float):
  """x [T, ..., n] (n even): channel i < n/2 is paired with channel i + n/2 and the pair turned by positions * base^(-2i/n)."""
  n = x.shape[-1]
  half = n // 2
  freq = float(base) ** (-2.0 * np.arange(half) / n)
  ang = np.asarray(positions, dtype=np.float64)[:, None] * freq  # [T, half]
  ang = ang.reshape((x.shape[0],) + (1,) * (x.ndim - 2) + (half,))
  c, s = np.cos(ang), np.sin(ang)
  a, b = x[..., :half], x[..., half:]
  return np.concatenate([a * c - b * s, b * c + a * s], axis=-1)


def distance_slopes(heads: int):
  return np.array([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)])


def softmax_rows(scores, visible, sink=None):
  """scores [T, T] (query, key), visible a boolean mask; `sink` adds exp(sink) to every row's denominator."""
  out = np.zeros_like(scores)
  for i in range(scores.shape[0]):
    idx = np.flatnonzero(visible[i])
    s = scores[i, idx]
    top = s.max() if sink is None else max(s.max(), sink)
    e = np.exp(s - top)
    den = e.sum() + (0.0 if sink is None else math.exp(sink - top))
    out[i, idx] = e / den
  return out


def window_mask(T: int, window: Optional[int]):
  i, j = np.arange(T)[:, None], np.arange(T)[None, :]
  m = j <= i
  if window:
    m &= (i - j) < window
  return m


def windowed_attention(h, p: Dict[str, np.ndarray], spec: dict, eps: float, shared_kv=None, fault: Optional[dict] = None):
  """Grouped-query softmax attention with per-head q/k norm, a linear distance penalty and a sliding window.  Returns the mixer's
  output and the (normed keys, values) it used, which a later layer may take over (`shared_kv`).  `fault` (tests of the tests):
  {"window_shift": n} widens the window by n keys."""
  T = h.shape[0]
  H, G, d, dv = int(spec["heads"]), int(spec["kv_heads"]), int(spec["dim"]), int(spec["vdim"])
  q = rms_unit((h @ p["q"].T).reshape(T, H, d), eps) * p["q.norm"]
  if shared_kv is None:
    k = rms_unit((h @ p["k"].T).reshape(T, G, d), eps) * p["k.norm"]
    v = (h @ p["v"].T).reshape(T, G, dv)
  else:
    k, v = shared_kv
  gate = sigmoid(h @ p["g"].T)  # [T, H]
  slopes = distance_slopes(H)
  mask = window_mask(T, int(spec["mask"]["size"]) + int((fault or {}).get("window_shift", 0)) if spec.get("mask") else None)
  dist = (np.arange(T)[:, None] - np.arange(T)[None, :]).astype(np.float64)
  out = np.zeros((T, H, dv))
  for hd in range(H):
    g = hd // (H // G)
    s = (q[:, hd] @ k[:, g].T) * float(spec["scale"]) - slopes[hd] * dist
    out[:, hd] = (softmax_rows(s, mask) @ v[:, g]) * gate[:, hd : hd + 1]
  return out.reshape(T, H * dv) @ p["o"].T, (k, v)


def latent_attention(h, p: Dict[str, np.ndarray], spec: dict, eps: float, fault: Optional[dict] = None):
  """Queries through a normed latent; keys and values expanded from a normed latent c; one rotated key part shared by the heads;
  causal softmax whose denominator also holds exp(sink) per head; a sigmoid gate per head.  `fault` (tests of the tests):
  {"horizon": n} hides keys more than n positions back, {"no_sink": True} leaves the sink out."""
  T = h.shape[0]
  H, d, dr, dv, rank = int(spec["heads"]), int(spec["dim"]), int(spec["rot_dim"]), int(spec["vdim"]), int(spec["kv_rank"])
  pos = np.arange(T)
  base = float(spec["rot"]["base"])
  cq = rms_unit(h @ p["dq"].T, eps) * p["dq.norm"]
  q = (cq @ p["uq"].T).reshape(T, H, d + dr)
  q_plain, q_rot = q[..., :d], rotate_half(q[..., d:], pos, base)
  kv = h @ p["dkv"].T
  c = rms_unit(kv[:, :rank], eps) * p["dkv.norm"]
  k_rot = rotate_half(kv[:, rank:], pos, base)  # [T, dr]
  k_plain = (c @ p["uk"].T).reshape(T, H, d)
  v = (c @ p["uv"].T).reshape(T, H, dv)
  gate = sigmoid(h @ p["g"].T)
  fault = fault or {}
  mask = window_mask(T, int(fault["horizon"]) + 1 if "horizon" in fault else None)
  out = np.zeros((T, H, dv))
  for hd in range(H):
    s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * float(spec["scale"])
    out[:, hd] = (softmax_rows(s, mask, sink=None if fault.get("no_sink") else float(p["sink"][hd])) @ v[:, hd]) * gate[:, hd : hd + 1]
  return out.reshape(T, H * dv) @ p["o"].T


DECAY_RATE = math.exp(-0.5)
UNIT_KEY_EPS = 1e-6


def delta_scan(r, k, v, w, a, state=None):
  """One head: r, k, w, a [T, d], v [T, dv].  S <- diag(w) S - (a u)(u^T S) + k v^T with u = k / sqrt(|k|^2 + 1e-6), both first
  terms from the old S; o = S^T r.  Returns o [T, dv] and the last S."""
  T, d = k.shape
  S = np.zeros((d, v.shape[1])) if state is None else state.copy()
  o = np.zeros((T, v.shape[1]))
  for t in range(T):
    u = k[t] / math.sqrt(float(k[t] @ k[t]) + UNIT_KEY_EPS)
    S = w[t][:, None] * S - np.outer(a[t] * u, u @ S) + np.outer(k[t], v[t])
    o[t] = S.T @ r[t]
  return o, S


def general_delta(h, p: Dict[str, np.ndarray], spec: dict, eps: float):
  T = h.shape[0]
  H, d = int(spec["heads"]), int(spec["dim"])
  r, k, v = ((h @ p[n].T).reshape(T, H, d) for n in ("r", "k", "v"))
  w = np.exp(-DECAY_RATE * sigmoid(np.tanh(h @ p["w1"].T) @ p["w2"].T + p["w0"])).reshape(T, H, d)
  a = sigmoid(h @ p["a"].T + p["a.b"]).reshape(T, H, d)
  o = np.zeros((T, H, d))
  for hd in range(H):
    o[:, hd], _ = delta_scan(r[:, hd], k[:, hd], v[:, hd], w[:, hd], a[:, hd])
  o = rms_unit(o, eps).reshape(T, H * d) * p["norm"] * sigmoid(h @ p["g"].T)
  return o @ p["o"].T


def sub(tensors: Dict[str, np.ndarray], prefix: str) -> Dict[str, np.ndarray]:
  return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(model: dict, tensors: Dict[str, np.ndarray], tokens: List[int], return_layers: bool = False, fault: Optional[dict] = None):
  """Logits [T, vocab] of one sequence (and the residual stream after every layer, [L, T, E])."""
  eps, groups = float(model["norm"]["eps"]), int(model["norm"]["groups"])
  m = float(model["residual_mult"])
  x = tensors["embed"][np.asarray(tokens)]
  kept, stream = {}, []
  for i, layer in enumerate(model["layers"]):
    pre = f"l{i}."
    h = group_norm(x, tensors[pre + "norm1"], groups, eps)
    conv = (lambda z, name: z + causal_conv(z, tensors[name])) if model.get("canon") else (lambda z, name: z)
    hm = conv(h, pre + "canon1")
    spec, p = layer["mixer"], sub(tensors, pre + "mix.")
    if layer["type"] == "attention":
      src = spec.get("kv_from")
      y, kept[i] = windowed_attention(hm, p, spec, eps, kept[int(src)] if src is not None else None, fault)
    elif layer["type"] == "latent_attention":
      y = latent_attention(hm, p, spec, eps, fault)
    elif layer["type"] == "general_delta":
      y = general_delta(hm, p, spec, eps)
    else:
      raise ValueError(layer["type"])
    if layer.get("mlp"):
      hf = conv(h, pre + "canon2")
      y = y + squared_relu_ff(hf, tensors[pre + "mlp.up"], tensors[pre + "mlp.down"])
    x = x + m * y
    stream.append(x.copy())
  n = group_norm(x, tensors["final.norm"], groups, eps)
  z = (n @ tensors["embed"].T) * float(model.get("logit_scale", 1.0))
  cap = float(model.get("logit_softcap") or 0.0)
  if cap > 0.0:
    z = cap * np.tanh(z / cap)
  return (z, np.stack(stream)) if return_layers else z


def bf16_values(x):
  """x rounded to values that bfloat16 holds exactly (float64 array)."""
  import torch

  return torch.from_numpy(np.asarray(x, dtype=np.float32)).to(torch.bfloat16).to(torch.float64).numpy()


def random_model(model: dict, seed: int = 0, rank: int = 6) -> Dict[str, np.ndarray]:
  """Random weights by the stored names, already rounded to bfloat16 values.  `rank`: the decay's low rank of general_delta layers."""
  g = np.random.Generator(np.random.PCG64(seed))
  E, V = int(model["width"]), int(model["vocab"])
  taps = int(model["canon"]["taps"]) if model.get("canon") else 0
  t: Dict[str, np.ndarray] = {}
  rn = lambda *shape, std=1.0, mean=0.0: bf16_values(g.normal(mean, std, size=shape))
  lin = lambda n, k: rn(n, k, std=1.0 / math.sqrt(k))
  t["embed"], t["final.norm"] = rn(V, E), rn(E, std=0.2, mean=1.0)
  for i, layer in enumerate(model["layers"]):
    p, q, m = f"l{i}.", f"l{i}.mix.", layer["mixer"]
    t[p + "norm1"] = rn(E, std=0.2, mean=1.0)
    if taps:
      t[p + "canon1"] = rn(E, taps, std=0.4)
    if layer["type"] == "attention":
      H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
      t[q + "q"], t[q + "q.norm"], t[q + "g"], t[q + "o"] = lin(H * d, E), rn(d, std=0.3, mean=1.5), lin(H, E), lin(E, H * dv)
      if m.get("kv_from") is None:
        t[q + "k"], t[q + "k.norm"], t[q + "v"] = lin(G * d, E), rn(d, std=0.3, mean=1.5), lin(G * dv, E)
    elif layer["type"] == "latent_attention":
      H, d, dr, dv, qr, kr = (int(m[k]) for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"))
      t[q + "dq"], t[q + "dq.norm"], t[q + "uq"] = lin(qr, E), rn(qr, std=0.3, mean=1.5), lin(H * (d + dr), qr)
      t[q + "dkv"], t[q + "dkv.norm"] = lin(kr + dr, E), rn(kr, std=0.3, mean=1.5)
      t[q + "uk"], t[q + "uv"], t[q + "sink"] = lin(H * d, kr), lin(H * dv, kr), rn(H, std=1.5)
      t[q + "g"], t[q + "o"] = lin(H, E), lin(E, H * dv)
    else:
      H, d = int(m["heads"]), int(m["dim"])
      for n in ("r", "k", "v", "g", "a"):
        t[q + n] = lin(H * d, E)
      t[q + "a.b"], t[q + "w1"], t[q + "w2"], t[q + "w0"] = rn(H * d, std=0.5), lin(rank, E), rn(H * d, rank, std=1.0), rn(H * d, std=1.0)
      t[q + "norm"], t[q + "o"] = rn(H * d, std=0.2, mean=1.0), lin(E, H * d)
    if layer.get("mlp"):
      F = int(layer["mlp"]["ff"])
      t[p + "mlp.up"], t[p + "mlp.down"] = lin(F, E), lin(E, F)
      if taps:
        t[p + "canon2"] = rn(E, taps, std=0.4)
  return t
