"""A plain float64 restatement of the Ligidra design, one function per mechanism, for the tests.

Nothing here is shared with the engine: numpy only, whole sequences, O(n^2) attention written as loops over query positions, the
recurrence as the token loop that defines it.  `tensors` maps the stored names to float64 arrays (integer tables stay integers),
`model` is the config.json dict.  Notation: E width, T tokens of one sequence, H heads, G key heads, d per-head key size, dv
per-head value size, P tokens of a pooled block, W the window.

A layer:  h = rms(x) * n1;  x <- x + mixer(shift(h));  x <- x + ff(rms(x) * n2);  x <- x + unit(side(x, token)) * ns.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np

UNIT_EPS = 1e-6  # inside the root of the recurrences' unit vectors


def sigmoid(z):
  return 1.0 / (1.0 + np.exp(-z))


def silu(z):
  return z * sigmoid(z)


def softplus(z):
  return np.logaddexp(0.0, z)


def gelu_tanh(z):
  return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z**3)))


def rms_unit(x, eps):
  """x / sqrt(mean(x^2) + eps) over the last axis."""
  return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, w, eps):
  return rms_unit(x, eps) * w


def token_shift(h, mu):
  """h [T, E]: every row moves towards the row before it (zeros before the first), channel by channel: h + (h_prev - h) * mu."""
  prev = np.concatenate([np.zeros((1, h.shape[1])), h[:-1]], axis=0)
  return h + (prev - h) * mu


def scaled_frequencies(dims: int, base: float, scaling: Optional[dict] = None):
  """Radians per position of pair i < dims / 2: base^(-2i / dims); with `scaling`, long wavelengths are slowed: a wavelength above
  original / low by `factor`, one below original / high not at all, the ones between by a blend that is linear in original / wavelength."""
  f = float(base) ** (-2.0 * np.arange(dims // 2) / dims)
  if not scaling:
    return f
  factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
  out = np.empty_like(f)
  for i, fi in enumerate(f):
    wavelength = 2.0 * math.pi / fi
    if wavelength < orig / high:
      out[i] = fi
    elif wavelength > orig / low:
      out[i] = fi / factor
    else:
      s = (orig / wavelength - low) / (high - low)
      out[i] = (1.0 - s) * fi / factor + s * fi
  return out


def rotate_pairs(x, positions, freq):
  """x [T, heads, n]: the channel pairs (2i, 2i + 1), i < len(freq), turn by positions * freq[i]; the other channels pass."""
  out = x.copy()
  ang = np.asarray(positions, dtype=np.float64)[:, None] * freq  # [T, pairs]
  c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
  n = 2 * len(freq)
  a, b = x[..., 0:n:2], x[..., 1:n:2]
  out[..., 0:n:2] = a * c - b * s
  out[..., 1:n:2] = b * c + a * s
  return out


def soft_cap(s, cap):
  return cap * np.tanh(s / cap) if cap else s


def visible(i: int, window: int, pool: int):
  """What the query at position i sees: (token positions, pooled block numbers).  Tokens j with 0 <= i - j < window (window 0:
  all j <= i); blocks b of `pool` tokens whose last token b * pool + pool - 1 is at most i - window."""
  lo = max(0, i - window + 1) if window else 0
  blocks = []
  if window and pool:
    b = 0
    while b * pool + pool - 1 <= i - window:
      blocks.append(b)
      b += 1
  return list(range(lo, i + 1)), blocks


def pooled_window_attention(q, k, v, scale, cap, window, pool, sink, hooks=None):
  """q [T, H, d] and k [T, G, d] (after norm and rotation), v [T, G, dv] -> [T, H, dv].  One softmax over the visible tokens and
  the visible blocks' mean keys, with exp(sink_h) in the denominator besides.  `hooks` (tests): {"window": +-1, "blocks": +-1,
  "no_sink": True} make a deliberate fault."""
  T, H, d = q.shape
  G, dv = k.shape[1], v.shape[2]
  head_of = np.arange(H) // (H // G)  # the key head of every query head
  hooks = hooks or {}
  out = np.zeros((T, H, dv))
  for i in range(T):
    toks, blocks = visible(i, window + hooks.get("window", 0) if window else 0, pool)
    if hooks.get("blocks"):
      blocks = list(range(max(0, len(blocks) + hooks["blocks"])))
    keys = np.stack([k[j] for j in toks] + [k[b * pool : (b + 1) * pool].mean(axis=0) for b in blocks])  # [n, G, d]
    vals = np.stack([v[j] for j in toks] + [v[b * pool : (b + 1) * pool].mean(axis=0) for b in blocks])  # [n, G, dv]
    s = soft_cap(np.einsum("hd,nhd->hn", q[i], keys[:, head_of]) * scale, cap)                           # [H, n]
    m = s.max(axis=1)
    if sink is not None:
      m = np.maximum(m, sink)
    p = np.exp(s - m[:, None])
    denom = p.sum(axis=1)
    if sink is not None and not hooks.get("no_sink"):
      denom = denom + np.exp(sink - m)
    out[i] = np.einsum("hn,nhc->hc", p, vals[:, head_of]) / denom[:, None]
  return out


def short_conv(x, w):
  """x [T, C], w [C, taps]: out[t] = sum_j w[:, j] * x[t - (taps - 1) + j]; rows before the sequence count as zero."""
  T, C = x.shape
  taps = w.shape[1]
  padded = np.concatenate([np.zeros((taps - 1, C)), x], axis=0)
  out = np.zeros_like(x)
  for j in range(taps):
    out += padded[j : j + T] * w[:, j]
  return out


def unit_vectors(x):
  return x / np.sqrt(np.sum(x * x, axis=-1, keepdims=True) + UNIT_EPS)


def gated_delta_scan(q, k, v, decay, beta, state=None):
  """One head.  q, k [T, d], v [T, dv], decay [T, d] (or [T, 1]), beta [T].  S [d, dv] from zero:
  S <- decay * S (row by row); u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
  T, d = q.shape
  dv = v.shape[1]
  S = np.zeros((d, dv)) if state is None else state.copy()
  o = np.zeros((T, dv))
  for t in range(T):
    S = S * np.broadcast_to(decay[t], (d,))[:, None]
    u = beta[t] * (v[t] - S.T @ k[t])
    S = S + np.outer(k[t], u)
    o[t] = S.T @ q[t]
  return o, S


def attention_mixer(h, t: Dict[str, np.ndarray], p: str, m: dict, eps: float, kv=None, hooks=None):
  """-> (output [T, E], (k, v) as cached).  `kv`: the cached keys and values of the layer named by kv_from."""
  T = h.shape[0]
  H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
  pos = np.arange(T)
  rot = m.get("rot")
  freq = scaled_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling")) if rot else np.zeros(0)
  q = rms_norm(h @ t[p + "q"].T, t[p + "q.norm"], eps).reshape(T, H, d)
  q = rotate_pairs(q, pos, freq)
  if kv is None:
    k = rms_norm(h @ t[p + "k"].T, t[p + "k.norm"], eps).reshape(T, G, d)
    k = rotate_pairs(k, pos, freq)
    v = (h @ t[p + "v"].T).reshape(T, G, dv)
  else:
    k, v = kv
  mask = m.get("mask") or {}
  o = pooled_window_attention(q, k, v, float(m["scale"]), float(m.get("softcap") or 0.0), int(mask.get("size") or 0), int(mask.get("pool") or 0),
                              t[p + "sink"] if (p + "sink") in t else None, hooks)
  return o.reshape(T, H * dv) @ t[p + "o"].T, (k, v)


def delta_mixer(h, t: Dict[str, np.ndarray], p: str, m: dict, eps: float, per_channel: bool):
  T = h.shape[0]
  H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
  rep = H // G
  q = unit_vectors(silu(short_conv(h @ t[p + "q"].T, t[p + "q.conv"])).reshape(T, G, d)) * d**-0.5
  k = unit_vectors(silu(short_conv(h @ t[p + "k"].T, t[p + "k.conv"])).reshape(T, G, d))
  v = silu(short_conv(h @ t[p + "v"].T, t[p + "v.conv"])).reshape(T, H, dv)
  beta = sigmoid(h @ t[p + "b"].T)  # [T, H]
  rate = np.exp(t[p + "A_log"])     # [H]
  if per_channel:
    z = ((h @ t[p + "a1"].T) @ t[p + "a2"].T + t[p + "dt_bias"]).reshape(T, H, d)
    decay = np.exp(-rate[None, :, None] * softplus(z))
    gate = sigmoid((h @ t[p + "g1"].T) @ t[p + "g2"].T).reshape(T, H, dv)
  else:
    decay = np.exp(-rate * softplus(h @ t[p + "a"].T + t[p + "dt_bias"]))[:, :, None]  # [T, H, 1]
    gate = silu(h @ t[p + "g"].T).reshape(T, H, dv)
  o = np.zeros((T, H, dv))
  for hh in range(H):
    o[:, hh], _ = gated_delta_scan(q[:, hh // rep], k[:, hh // rep], v[:, hh], decay[:, hh], beta[:, hh])
  o = rms_unit(o, eps) * t[p + "norm"] * gate
  return o.reshape(T, H * dv) @ t[p + "o"].T


def gated_expert(h, t, p):
  return (silu(h @ t[p + "gate"].T) * (h @ t[p + "up"].T)) @ t[p + "down"].T


def route(z, top: int):
  """z [T, experts] -> (chosen [T, top], weights [T, top]): softmax over all experts, the `top` largest, their scores as they are."""
  s = np.exp(z - z.max(axis=-1, keepdims=True))
  s /= s.sum(axis=-1, keepdims=True)
  chosen = np.argsort(-s, axis=-1, kind="stable")[:, :top]
  return chosen, np.take_along_axis(s, chosen, axis=-1)


def moe_ff(h, t, p, f: dict):
  n, top = int(f["router"]["experts"]), int(f["router"]["top"])
  chosen, w = route(h @ t[p + "router"].T, top)
  outs = [gated_expert(h, t, f"{p}e{e}.") for e in range(n)]
  y = np.zeros_like(outs[0])
  for r in range(h.shape[0]):
    for c in range(top):
      y[r] += w[r, c] * outs[chosen[r, c]][r]
  if f.get("shared"):
    y = y + gated_expert(h, t, p + "shared.")
  return y


def side_input(x, tokens, t, i: int, dim: int, eps: float):
  """What layer i adds after its feed-forward: unit(proj(gelu_tanh(gate x) * e)) * norm, e = the layer's part of the tokens' rows."""
  e = t["side.embed"][np.asarray(tokens), i * dim : (i + 1) * dim]
  y = (gelu_tanh(x @ t[f"l{i}.side.gate"].T) * e) @ t[f"l{i}.side.proj"].T
  return rms_unit(y, eps) * t[f"l{i}.side.norm"]


def forward(model: dict, t: Dict[str, np.ndarray], tokens, hooks=None, return_layers: bool = False):
  """Logits [T, vocab] of one sequence (float64)."""
  eps = float(model["norm"]["eps"])
  tokens = np.asarray(tokens)
  x = rms_norm(t["embed"][tokens], t["embed.norm"], eps)
  side = model.get("token_side")
  caches: List[Optional[tuple]] = []
  layers = []
  for i, l in enumerate(model["layers"]):
    p, m = f"l{i}.mix.", l["mixer"]
    h = token_shift(rms_norm(x, t[f"l{i}.norm1"], eps), t[f"l{i}.shift"])
    if l["type"] == "attention":
      src = m.get("kv_from")
      y, kv = attention_mixer(h, t, p, m, eps, None if src is None else caches[int(src)], (hooks or {}).get(i))
      caches.append(kv if src is None else None)
    else:
      y = delta_mixer(h, t, p, m, eps, l["type"] == "channel_delta")
      caches.append(None)
    x = x + y
    if l.get("mlp"):
      x = x + moe_ff(rms_norm(x, t[f"l{i}.norm2"], eps), t, f"l{i}.mlp.", l["mlp"])
    if side:
      x = x + side_input(x, tokens, t, i, int(side["dim"]), eps)
    layers.append(x.copy())
  logits = rms_norm(x, t["final.norm"], eps) @ t["embed"].T
  return (logits, np.stack(layers)) if return_layers else logits


# -- random models (tests) -----------------------------------------------------------------------------------------------------


def bf16_values(x):
  """float64 array -> the nearest bfloat16 values (round to nearest even), as float64."""
  a = np.ascontiguousarray(np.asarray(x, dtype=np.float32))
  bits = a.view(np.uint32).astype(np.uint64)
  bits = ((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
  return bits.view(np.float32).astype(np.float64).reshape(np.shape(x))


def random_model(model: dict, seed: int = 0, rank: int = 6) -> Dict[str, np.ndarray]:
  """Random weights by the stored names, already bfloat16 values.  `rank`: the low ranks of channel_delta layers."""
  g = np.random.Generator(np.random.PCG64(seed))
  E, V, n = int(model["width"]), int(model["vocab"]), len(model["layers"])
  sd = int((model.get("token_side") or {}).get("dim") or 0)
  t: Dict[str, np.ndarray] = {}
  rn = lambda *shape, std=1.0, mean=0.0: bf16_values(g.normal(mean, std, size=shape))
  un = lambda *shape, lo=0.0, hi=1.0: bf16_values(g.uniform(lo, hi, size=shape))
  lin = lambda a, b: rn(a, b, std=1.0 / math.sqrt(b))
  t["embed"], t["embed.norm"], t["final.norm"] = rn(V, E), rn(E, std=0.2, mean=1.0), rn(E, std=0.2, mean=1.0)
  if sd:
    t["side.embed"] = rn(V, n * sd)
  for i, layer in enumerate(model["layers"]):
    p, q, m = f"l{i}.", f"l{i}.mix.", layer["mixer"]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    t[p + "norm1"], t[p + "shift"] = rn(E, std=0.2, mean=1.0), un(E)
    if layer["type"] == "attention":
      t[q + "q"], t[q + "q.norm"], t[q + "sink"], t[q + "o"] = lin(H * d, E), rn(H * d, std=0.3, mean=1.5), rn(H, std=1.0), lin(E, H * dv)
      if m.get("kv_from") is None:
        t[q + "k"], t[q + "k.norm"], t[q + "v"] = lin(G * d, E), rn(G * d, std=0.3, mean=1.5), lin(G * dv, E)
    else:
      taps = int(m["conv"])
      t[q + "q"], t[q + "k"], t[q + "v"], t[q + "b"] = lin(G * d, E), lin(G * d, E), lin(H * dv, E), lin(H, E)
      t[q + "q.conv"], t[q + "k.conv"], t[q + "v.conv"] = rn(G * d, taps, std=0.6), rn(G * d, taps, std=0.6), rn(H * dv, taps, std=0.6)
      t[q + "A_log"], t[q + "norm"], t[q + "o"] = un(H, lo=-3.0, hi=0.5), rn(dv, std=0.2, mean=1.0), lin(E, H * dv)
      if layer["type"] == "channel_delta":
        t[q + "a1"], t[q + "a2"], t[q + "dt_bias"] = lin(rank, E), rn(H * d, rank, std=1.0), rn(H * d, std=1.0)
        t[q + "g1"], t[q + "g2"] = lin(rank + 1, E), rn(H * dv, rank + 1, std=1.0)
      else:
        t[q + "a"], t[q + "dt_bias"], t[q + "g"] = lin(H, E), rn(H, std=1.0), lin(H * dv, E)
    f = layer.get("mlp")
    if f:
      t[p + "norm2"] = rn(E, std=0.2, mean=1.0)
      names = [f"{p}mlp.e{e}." for e in range(int(f["router"]["experts"]))] + ([p + "mlp.shared."] if f.get("shared") else [])
      for name in names:
        F = int(f["shared"]["ff"]) if name.endswith("shared.") else int(f["expert"]["ff"])
        t[name + "gate"], t[name + "up"], t[name + "down"] = lin(F, E), lin(F, E), lin(E, F)
      t[p + "mlp.router"] = rn(int(f["router"]["experts"]), E, std=3.0 / math.sqrt(E))
    if sd:
      t[p + "side.gate"], t[p + "side.proj"], t[p + "side.norm"] = lin(sd, E), lin(E, sd), rn(E, std=0.1, mean=0.4)
  return t


def closest_router_gap(model: dict, t: Dict[str, np.ndarray], tokens) -> float:
  """The smallest difference, over all rows and routed layers of a sequence, between the score of the last expert that is chosen
  and the first that is not: a test whose gap is tiny rests on a close call and should take another seed."""
  gaps = [1.0]
  eps = float(model["norm"]["eps"])
  tokens = np.asarray(tokens)
  x = rms_norm(t["embed"][tokens], t["embed.norm"], eps)
  side = model.get("token_side")
  caches: List[Optional[tuple]] = []
  for i, l in enumerate(model["layers"]):
    p, m = f"l{i}.mix.", l["mixer"]
    h = token_shift(rms_norm(x, t[f"l{i}.norm1"], eps), t[f"l{i}.shift"])
    if l["type"] == "attention":
      src = m.get("kv_from")
      y, kv = attention_mixer(h, t, p, m, eps, None if src is None else caches[int(src)])
      caches.append(kv if src is None else None)
    else:
      y = delta_mixer(h, t, p, m, eps, l["type"] == "channel_delta")
      caches.append(None)
    x = x + y
    f = l.get("mlp")
    if f:
      hn = rms_norm(x, t[f"l{i}.norm2"], eps)
      z = hn @ t[f"l{i}.mlp.router"].T
      s = np.exp(z - z.max(axis=-1, keepdims=True))
      s = np.sort(s / s.sum(axis=-1, keepdims=True), axis=-1)[:, ::-1]
      top = int(f["router"]["top"])
      if top < s.shape[1]:
        gaps.append(float((s[:, top - 1] - s[:, top]).min()))
      x = x + moe_ff(hn, t, f"l{i}.mlp.", f)
    if side:
      x = x + side_input(x, tokens, t, i, int(side["dim"]), eps)
  return min(gaps)
