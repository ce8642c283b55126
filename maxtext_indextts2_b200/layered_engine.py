"""MaxEngine for the layered designs (``pyconfig.LAYERED_BLOCKS``): the same engine API over ``mtx_layered_*``.

A layered model is a list of layer descriptors (sizes, windows, sublayers that differ per layer), and its step takes a ragged
batch: portions of prompts beside single decoded tokens, every row tagged with its page group and position.  So the three
phases of the reference's engine are one device function here:

* ``prefill``  -- the prompt's rows of ONE page group, written straight into that group's pages (no staging plane, no copy
  at ``insert``); with ``existing_prefix`` the group simply grows (chunked prefill);
* ``generate`` -- one row per decode slot (empty slots write the never-handed-out page 0);
* ``step``     -- any mix of both, the entry point of continuous batching with chunked prompts and of ``trace_run``.

The cache is the page manager's (``page_manager.PageManager``: pages handed out lowest index first, given back by
``release_pages``); sampling is the framework's sampler on the step's logits (``mtx_sample_rows``).  Everything computed
runs in ``libmtx_b200.so``; this file moves descriptors.
"""

from __future__ import annotations

import ctypes
from typing import Any, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib
from . import page_manager
from . import params as params_lib
from .maxengine import ExistingPrefix, MaxEngine, ResultTokens  # noqa: F401  (same result types)

_MIXERS = {"window_sigmoid": _lib.MIXER_WINDOW_SIGMOID, "composite": _lib.MIXER_COMPOSITE}
_NORMS = {"out_gain": _lib.NORM_OUT_GAIN, "sandwich": _lib.NORM_SANDWICH, "parallel": _lib.NORM_PARALLEL, "pre": _lib.NORM_PRE}
_FF_KINDS = {"none": _lib.FF_GELU_GATED, "gelu": _lib.FF_GELU_GATED, "clamped": _lib.FF_CLAMPED_GATED, "moe": _lib.FF_MOE, "relu2": _lib.FF_RELU2}
_RECURRENCES = {"gla": _lib.REC_GLA, "mlstm": _lib.REC_MLSTM, "delta": _lib.REC_DELTA, "gdelta": _lib.REC_GDELTA}
QUERY_TILE_ROWS = 16  # rows of one query tile of the attention kernels (csrc/window_attention_mma.cuh, csrc/softmax_attention.cuh)

_LAYER_MATS = ("wqkv", "wo", "w_gate_up", "w_down", "w_in")
_LAYER_VECS = ("bqkv", "q_norm", "k_norm", "dist_bias", "head_bias", "talk", "norm1", "norm1b", "norm2", "norm2b", "add_vector", "b_in", "bo",
               "conv1", "conv2")
_ATTN_VECS = ("q_norm", "k_norm", "slopes", "sink")
_LATENT_MATS = ("w_uq", "w_uk_t", "w_uv")
_LATENT_VECS = ("q_norm", "kv_norm", "sink")
_REC_VECS = ("decay_up_t", "decay_bias", "gate_bias", "out_norm", "conv_w", "a_log")
_REC_MATS = ("w_gate_up", "decay_up2")
_SIDE_MATS = ("gate", "proj")
_SIDE_VECS = ("norm",)
_MOE_MATS = ("w_router", "w_gate_up", "w_down", "shared_gate_up", "shared_down")
_MOE_VECS = ("correction",)


def design_module(config):
  """The module that knows the design named by config.decoder_block."""
  if config.decoder_block == "kifusun":
    from . import kifusun

    return kifusun
  if config.decoder_block == "gugidra":
    from . import gugidra

    return gugidra
  if config.decoder_block == "ginodra":
    from . import ginodra

    return ginodra
  if config.decoder_block == "ligidra":
    from . import ligidra

    return ligidra
  raise ValueError(f"decoder_block={config.decoder_block!r} is not a layered design")


class LayeredParams:
  """Device-resident weights of a layered model: one entry per layer RUN of the plan (a layer that runs several times is listed
  once per run; the runs share the device copy of every tensor that is the same host tensor)."""

  def __init__(self, plan: dict, config, device):
    fp32 = config.dtype == "float32"
    wt = torch.float32 if fp32 else torch.bfloat16
    self.float32 = fp32
    self.keep: List[torch.Tensor] = []
    moved = {}  # id(host tensor) -> (host tensor, device tensor): shared weights are uploaded once

    def put(t, dtype):
      if t is None:
        return None
      hit = moved.get((id(t), dtype))
      if hit is not None:
        return hit[1]
      d = t.to(device=device, dtype=dtype).contiguous()
      moved[(id(t), dtype)] = (t, d)
      self.keep.append(d)
      return d

    mat = lambda t: put(t, wt)
    vec = lambda t: put(t, torch.float32)

    def pack(src, mats, vecs):
      d = dict(src)
      for k in mats:
        if k in d:
          d[k] = mat(d[k])
      for k in vecs:
        if k in d:
          d[k] = vec(d[k])
      return d

    self.embedding, self.head = mat(plan["embedding"]), mat(plan["head"])
    self.final_gain, self.embed_scale = float(plan["final_gain"]), float(plan["embed_scale"])
    self.final_norm = vec(plan.get("final_norm"))
    self.logit_softcap = float(plan.get("logit_softcap") or 0.0)
    self.logit_scale = float(plan.get("logit_scale") or 1.0)
    self.norm_groups = int(plan.get("norm_groups") or 0)
    self.embed_norm = vec(plan.get("embed_norm"))
    self.side_embed = mat(plan.get("side_embed"))
    self.layers = []
    for lp in plan["layers"]:
      d = pack(lp, _LAYER_MATS, _LAYER_VECS)
      if d.get("attn"):
        d["attn"] = pack(d["attn"], (), _ATTN_VECS)
        d["attn"]["rot_freq"] = put(d["attn"].get("rot_freq"), torch.float64)  # (the rotation's frequencies stay float64)
      if d.get("latent"):
        d["latent"] = pack(d["latent"], _LATENT_MATS, _LATENT_VECS)
        d["latent"]["rot_freq"] = put(d["latent"].get("rot_freq"), torch.float64)
      if d.get("rec"):
        d["rec"] = pack(d["rec"], _REC_MATS, _REC_VECS)
      if d.get("side"):
        d["side"] = pack(d["side"], _SIDE_MATS, _SIDE_VECS)
      if d.get("moe"):
        d["moe"] = pack(d["moe"], _MOE_MATS, _MOE_VECS)
      self.layers.append(d)

  def nbytes(self) -> int:
    return sum(t.numel() * t.element_size() for t in self.keep)


class LayeredEngine(MaxEngine):
  """``MaxEngine(config)`` returns this class when ``config.decoder_block`` is a layered design."""

  prompt_and_decode_share_pages = True  # no prefill segment + AR ring: a sequence is one page group that grows

  def __init__(self, config, devices: Any = None, use_cuda_graph: bool = True, vocab_shard: Optional[tuple] = None, gather: Any = None):
    if vocab_shard is not None or int(config.vocab_parallelism) != 1:
      raise ValueError("a layered model runs with vocab_parallelism=1")
    self.config = config
    self.device = _lib.require_cuda()
    self.lib = _lib.load()
    self.use_cuda_graph = use_cuda_graph
    self._handle = ctypes.c_void_p()
    self._params: Optional[LayeredParams] = None
    self._state = None
    self._paged, self._page_on_device, self._page_host_stale = True, False, False
    self.page_manager = page_manager.PageManager(config)
    self.page_state = self.page_manager.get_initial_page_state()
    B = self.max_concurrent_decodes
    self._max_rows = max(int(config.max_step_rows), B)
    dev, i32 = self.device, torch.int32
    self._tokens = torch.zeros(B, 1, dtype=i32, device=dev)
    self._next_pos = torch.zeros(B, 1, dtype=i32, device=dev)
    self._generated = torch.zeros(B, 1, dtype=i32, device=dev)
    self._active = torch.zeros(B, 1, dtype=i32, device=dev)
    self._result = torch.zeros(B, 3, dtype=i32, device=dev)
    self._log_prob = torch.zeros(B, 1, dtype=torch.float32, device=dev) if config.return_log_prob else None
    self._rng_state = torch.zeros(4, dtype=i32, device=dev)
    self._slot_ids = torch.arange(B, dtype=i32, device=dev)
    MP = self.page_manager.max_pages_per_group
    # (row B of the map stays zero: rows of empty slots are parked in group B, whose keys land on the never-handed-out page 0
    # and whose recurrent state nobody reads)
    self._page_map_dev = torch.zeros(B + 1, MP, dtype=i32, device=dev)
    self._uploaded_map = None
    # one pinned staging buffer per step: [token | group | pos | want | query tiles | runs] rows
    self._desc_host = torch.zeros(6 * self._max_rows + 16, dtype=i32).pin_memory()
    self._desc_dev = torch.zeros(6 * self._max_rows + 16, dtype=i32, device=dev)
    self._decode_tiles = torch.arange(B + 1, dtype=i32, device=dev)  # a decode step: every row is its own query tile and run
    self._decode_groups = torch.arange(B, dtype=i32, device=dev)
    self._states: List[tuple] = []
    self._needs_runs = False
    self._sample_scratch = torch.zeros(5 * max(B, 1), dtype=torch.float32, device=dev)
    self._first_token = torch.zeros(1, dtype=i32, device=dev)
    self._first_log_prob = torch.zeros(1, dtype=torch.float32, device=dev)
    self._logits = None
    self._pools: List[Tuple[torch.Tensor, torch.Tensor]] = []
    self._ws = None

  def __del__(self):
    try:
      if self._handle:
        self.lib.mtx_layered_destroy(self._handle)
    except Exception:  # pragma: no cover - interpreter shutdown
      pass

  # -- weights ------------------------------------------------------------------------------------

  def load_params(self, params: Any = None, rng: Any = None, on_device_init: bool = False, norm_jitter: float = 0.0) -> LayeredParams:
    """`params`: the design's tensors by their stored names (``params.load_model_dir``), a LayeredParams, or None: the folder
    ``config.model_dir`` if set, else random weights (made on the device with ``on_device_init``)."""
    cfg = self.config
    if isinstance(params, LayeredParams):
      lp = params
    else:
      design = design_module(cfg)
      if params is None:
        if cfg.model_dir:
          params = params_lib.load_model_dir(cfg.model_dir)
        else:
          params = design.random_tensors(cfg, seed=int(cfg.init_weights_seed), device=self.device if on_device_init else "cpu")
      lp = LayeredParams(design.model_plan(cfg, params), cfg, self.device)
    if lp.float32 != (cfg.dtype == "float32"):
      raise ValueError("these LayeredParams were packed for another dtype")
    self._create(lp)
    self._params = lp
    return lp

  def _create(self, lp: LayeredParams) -> None:
    cfg, dev = self.config, self.device
    if self._handle:
      self.lib.mtx_layered_destroy(self._handle)
      self._handle = ctypes.c_void_p()
    pm = self.page_manager
    ct = torch.float32 if lp.float32 else torch.bfloat16
    self._pools = []
    self._pooled = {}  # layer run -> (pooled keys, pooled values) of attention layers that see pooled blocks
    self._states = []  # per layer run: the recurrent state tensors [state slots, ...] (fp32), or ()
    descs = (_lib.LayerDesc * len(lp.layers))()
    ptr = lambda t: t.data_ptr() if t is not None else None
    slots = self.max_concurrent_decodes + 1  # (+ the parking slot of rows that belong to no live sequence)

    def pools(G, d, dv):
      kp = torch.zeros(G, pm.num_pages, pm.tokens_per_page, d, dtype=ct, device=dev)
      vp = torch.zeros(G, pm.num_pages, pm.tokens_per_page, dv, dtype=ct, device=dev)
      self._pools.append((kp, vp))
      return kp, vp

    for i, l in enumerate(lp.layers):
      d = descs[i]
      d.mixer = _MIXERS[l["mixer"]]
      d.norm_style = _NORMS[l.get("norm_style", "out_gain")]
      d.ff_kind = _FF_KINDS[l.get("ff_kind", "gelu")]
      d.ff = int(l.get("ff", 0))
      states = ()
      if l["mixer"] == "window_sigmoid":
        kp, vp = pools(l["kv_heads"], l["dim"], l["vdim"])
        for k in ("heads", "kv_heads", "dim", "vdim", "window", "value_mix"):
          setattr(d, k, int(l[k]))
        for k in ("scale", "softcap", "value_lambda", "gain1", "gain2"):
          setattr(d, k, float(l[k]))
        for k in ("wqkv", "bqkv", "q_norm", "k_norm", "dist_bias", "head_bias", "talk"):
          setattr(d, k, ptr(l[k]))
        d.k_pages, d.v_pages = kp.data_ptr(), vp.data_ptr()
      else:
        d.n_in, d.add_embedding, d.ff_limit = int(l["n_in"]), int(l.get("add_embedding", 0)), float(l.get("ff_limit", 0.0))
        for k in ("norm1", "norm1b", "norm2", "norm2b", "add_vector", "w_in", "b_in", "bo", "conv1", "conv2"):
          setattr(d, k, ptr(l.get(k)))
        a, r, m, lat = l.get("attn"), l.get("rec"), l.get("moe"), l.get("latent")
        d.conv_taps, d.residual_mult = int(l.get("conv_taps", 0)), float(l.get("residual_mult", 1.0))
        if d.conv_taps > 1:  # the ring of a sequence's last normed rows, per state slot
          states += (torch.zeros(slots, d.conv_taps - 1, int(cfg.emb_dim), dtype=torch.float32, device=dev),)
          d.conv_state = states[-1].data_ptr()
        if a:
          if a.get("kv_from") is not None:  # the pools of an earlier layer, read as that layer writes them
            kp, vp = self._pools[int(a["kv_from"])]
            self._pools.append(())
          else:
            kp, vp = pools(a["kv_heads"], a["dim"], a["vdim"])
          for k in ("heads", "kv_heads", "dim", "vdim", "window", "rot_dims", "values_are_keys", "rot_half", "shared_kv", "head_gate"):
            setattr(d.attn, k, int(a.get(k, 0)))
          d.attn.scale, d.attn.out_scale = float(a["scale"]), float(a["out_scale"])
          d.attn.rot_freq, d.attn.k_pages, d.attn.v_pages = ptr(a["rot_freq"]), kp.data_ptr(), vp.data_ptr()
          for k in _ATTN_VECS:
            setattr(d.attn, k, ptr(a.get(k)))
          d.attn.softcap, d.attn.norm_whole = float(a.get("softcap") or 0.0), int(a.get("norm_whole", 0))
          P = int(a.get("pool") or 0)
          if P:  # one mean key / value per block of P tokens, in pools of their own on the same page map
            tpp = pm.tokens_per_page
            slots_pp = tpp // P if tpp % P == 0 else tpp
            src = a.get("kv_from")
            if src is not None and int(lp.layers[int(src)]["attn"].get("pool") or 0) == P:  # the layer whose cache is read fills them
              pk, pv = self._pooled[int(src)]
              d.attn.pool_shared = 1
            else:
              pk = torch.zeros(int(a["kv_heads"]), pm.num_pages, slots_pp, int(a["dim"]), dtype=ct, device=dev)
              pv = torch.zeros(int(a["kv_heads"]), pm.num_pages, slots_pp, int(a["vdim"]), dtype=ct, device=dev)
            self._pooled[i] = (pk, pv)
            d.attn.pool, d.attn.pool_slots, d.attn.kp_pages, d.attn.vp_pages = P, slots_pp, pk.data_ptr(), pv.data_ptr()
        elif lat:
          dl = int(lat["kv_rank"]) + int(lat["rot_dim"])
          kp = torch.zeros(1, pm.num_pages, pm.tokens_per_page, dl, dtype=ct, device=dev)  # [latent | rotated key part] per token
          self._pools.append((kp, kp))
          for k in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "rot_half"):
            setattr(d.latent, k, int(lat[k]))
          d.latent.scale, d.latent.pages = float(lat["scale"]), kp.data_ptr()
          for k in ("rot_freq",) + _LATENT_MATS + _LATENT_VECS:
            setattr(d.latent, k, ptr(lat.get(k)))
        else:
          self._pools.append(())
        if r:
          d.rec.kind = _RECURRENCES[r["kind"]]
          for k in ("heads", "dim", "vdim", "decay_rank", "gate_silu"):
            setattr(d.rec, k, int(r[k]))
          for k in ("q_scale", "tau", "gate_cap", "denom_eps", "out_scale"):
            setattr(d.rec, k, float(r[k]))
          d.rec.decay_rate, d.rec.key_eps = float(r.get("decay_rate", 0.0)), float(r.get("key_eps", 0.0))
          for k in ("decay_up_t", "decay_bias", "gate_bias", "out_norm"):
            setattr(d.rec, k, ptr(r.get(k)))
          H, dk, dv = int(r["heads"]), int(r["dim"]), int(r["vdim"])
          f32 = torch.float32
          if r["kind"] == "gdelta":
            d.rec.kv_heads, d.rec.conv_taps, d.rec.gate_rank = int(r["kv_heads"]), int(r["conv_taps"]), int(r.get("gate_rank", 0))
            for k in ("conv_w", "a_log", "w_gate_up"):
              setattr(d.rec, k, ptr(r.get(k)))
            d.rec.decay_up_t = ptr(r.get("decay_up2"))  # (in the matmul dtype, written twice along its inputs)
            if d.rec.conv_taps > 1:  # the ring of a sequence's last projection rows (q | k | v before the convolution), per state slot
              states += (torch.zeros(slots, d.rec.conv_taps - 1, 2 * int(r["kv_heads"]) * dk + H * dv, dtype=f32, device=dev),)
              d.rec.conv_state = states[-1].data_ptr()
          rec_states = (torch.zeros(slots, H, dv, dk, dtype=f32, device=dev),)
          d.rec.state_s = rec_states[0].data_ptr()
          if r["kind"] == "mlstm":
            rec_states += (torch.zeros(slots, H, dk, dtype=f32, device=dev), torch.zeros(slots, H, dtype=f32, device=dev))
            d.rec.state_n, d.rec.state_m = rec_states[1].data_ptr(), rec_states[2].data_ptr()
          states += rec_states
        if m:
          for k in ("experts", "top", "groups", "keep_groups", "ff", "shared_ff"):
            setattr(d.moe, k, int(m[k]))
          d.moe.limit, d.moe.shared_limit = float(m["limit"]), float(m["shared_limit"])
          for k in ("w_router", "correction", "w_gate_up", "w_down", "shared_gate_up", "shared_down"):
            setattr(d.moe, k, ptr(m.get(k)))
          for k in ("score_softmax", "plain_weights", "act_silu"):
            setattr(d.moe, k, int(m.get(k, 0)))
        sd = l.get("side")
        if sd:
          d.side_dim, d.side_col = int(sd["dim"]), int(sd["col"])
          d.side_gate, d.side_proj, d.side_norm = ptr(sd["gate"]), ptr(sd["proj"]), ptr(sd["norm"])
          d.side_gate_rows = int(sd["gate"].shape[0])
      for k in ("wo", "w_gate_up", "w_down"):
        setattr(d, k, ptr(l.get(k)))
      self._states.append(states)
    self._needs_runs = any(l["mixer"] == "composite" for l in lp.layers)
    self._pool_tensors = []  # every page pool once (a pool that serves two roles or two layers is one tensor)
    for pool in list(self._pools) + list(self._pooled.values()):
      for t in pool:
        if not any(t is u for u in self._pool_tensors):
          self._pool_tensors.append(t)
    c = _lib.LayeredConfig(
        num_layers=len(lp.layers), width=int(cfg.emb_dim), vocab=int(cfg.vocab_size), float32=1 if lp.float32 else 0,
        max_rows=self._max_rows, max_want=self._max_rows, num_groups=slots, num_pages=pm.num_pages,
        tokens_per_page=pm.tokens_per_page, max_pages_per_group=pm.max_pages_per_group, eps=float(cfg.normalization_layer_epsilon),
        embed_scale=lp.embed_scale, final_gain=lp.final_gain, embedding=lp.embedding.data_ptr(), head=lp.head.data_ptr(),
        final_norm=ptr(lp.final_norm), logit_softcap=lp.logit_softcap, norm_groups=lp.norm_groups, logit_scale=lp.logit_scale,
        embed_norm=ptr(lp.embed_norm), side_embed=ptr(lp.side_embed), side_width=int(lp.side_embed.shape[1]) if lp.side_embed is not None else 0)
    _lib.check(self.lib.mtx_layered_create(ctypes.byref(c), descs, ctypes.byref(self._handle)))
    ws = int(self.lib.mtx_layered_workspace_bytes(self._handle))
    self._ws = torch.empty(ws + 1024, dtype=torch.uint8, device=dev)
    base = (self._ws.data_ptr() + 1023) // 1024 * 1024
    _lib.check(self.lib.mtx_layered_bind(self._handle, ctypes.c_void_p(base), ws))
    self._logits_buf = torch.zeros(self._max_rows, int(cfg.vocab_size), dtype=torch.float32, device=dev)

  def _require_params(self, params) -> None:
    if self._params is None or (params is not None and params is not self._params):
      raise ValueError("pass the params returned by this engine's load_params")

  # -- state --------------------------------------------------------------------------------------

  def init_decode_state(self, rng: Any = None) -> dict:
    for t in (self._tokens, self._next_pos, self._generated, self._active, self._result):
      t.zero_()
    self._rng_state[0:1].zero_()
    self._seed(rng)
    self.page_state = self.page_manager.get_initial_page_state()
    self._uploaded_map = None
    B, V = self.max_concurrent_decodes, int(self.config.vocab_size)
    self._logits = torch.zeros(B, 1, V, dtype=torch.float32, device=self.device)
    self._state = {
        "logits": self._logits,
        "cache": {"key_pages": [p[0] for p in self._pools if p], "value_pages": [p[1] for p in self._pools if p and p[1] is not p[0]],
                  "recurrent_state": [t for st in self._states for t in st]},
        "next_pos": self._next_pos,
        "generated_tokens": self._generated,
        "tokens": self._tokens,
    }
    return self._state

  def _upload_page_map(self) -> None:
    ps = self.page_state
    if ps.page_map is not self._uploaded_map:
      self._page_map_dev[: ps.page_map.shape[0]].copy_(torch.from_numpy(ps.page_map))
      self._uploaded_map = ps.page_map

  def _upload_page_state(self) -> None:  # (MaxEngine.release_pages calls it for device-resident page states; nothing to do here)
    return

  def release_pages(self, slot: int) -> None:
    """The slot's pages go back to the pool.  Its row of the page map is cleared too, so that the row an empty slot still
    contributes to a decode step lands on page 0 (never handed out) and not on a page somebody else owns by then."""
    slot = int(slot)
    ps = self.page_manager.release_pages(page_state=self.page_state, page_group_id=slot)
    page_map = ps.page_map.copy()
    page_map[slot] = 0
    self.page_state = ps.replace(page_map=page_map)
    self._active[slot].zero_()
    self._next_pos[slot].zero_()
    for st in self._states:  # (a sequence that starts at position 0 starts from zero anyway; this keeps a freed slot clean)
      for t in st:
        t[slot].zero_()

  # -- the ragged step ----------------------------------------------------------------------------

  def _run(self, rows: int, token_ptr: int, group_ptr: int, pos_ptr: int, n_want: int, want_ptr: int, logits: Optional[torch.Tensor],
           n_tiles: int = 0, tiles_ptr: Optional[int] = None, graph: bool = False, n_runs: int = 0, runs_ptr: Optional[int] = None) -> None:
    b = _lib.RaggedBatch(rows=rows, token=token_ptr, group=group_ptr, pos=pos_ptr, page_map=self._page_map_dev.data_ptr(), n_want=n_want,
                         want_rows=want_ptr if n_want else None, logits=logits.data_ptr() if n_want else None,
                         n_tiles=n_tiles, tile_row0=tiles_ptr if n_tiles else None, n_runs=n_runs, run_row0=runs_ptr if n_runs else None)
    fn = self.lib.mtx_layered_step_graph if graph else self.lib.mtx_layered_step
    _lib.check(fn(self._handle, ctypes.byref(b), self._stream()))

  def step(self, entries: Sequence[Tuple[int, Sequence[int], Sequence[int]]]) -> torch.Tensor:
    """One mixed batch.  `entries`: (slot, the sequence's next tokens, indices among them whose logits are wanted).  Every
    sequence grows by its tokens (pages are reserved as needed; ValueError when the pool is exhausted); returns the wanted
    logits [n, vocab] (fp32, on the device) in the order of the entries.  Steps longer than max_step_rows run in slices."""
    self._require_params(None)
    B, V = self.max_concurrent_decodes, int(self.config.vocab_size)
    tok, grp, pos, want, runs = [], [], [], [], []
    ps = self.page_state
    seen = set()
    for slot, tokens, wanted in entries:
      slot = int(slot)
      if not 0 <= slot < B or slot in seen:
        raise ValueError(f"slot {slot}: outside [0, {B}) or twice in one step")
      seen.add(slot)
      n = len(tokens)
      if n == 0:
        continue
      start = int(ps.sequence_lengths[slot])
      new = self.page_manager.extend_pages(ps, slot, start + n)
      if int(new.sequence_lengths[slot]) != start + n:
        raise ValueError(f"slot {slot}: the page pool cannot hold {start + n} tokens")
      ps = new
      base = len(tok)
      runs.append((base, base + n))
      tok.extend(int(t) for t in tokens)
      grp.extend([slot] * n)
      pos.extend(range(start, start + n))
      for w in wanted:
        if not 0 <= int(w) < n:
          raise ValueError(f"slot {slot}: wanted index {w} outside its {n} tokens")
        want.append(base + int(w))
    self.page_state = ps
    self._upload_page_map()
    rows = len(tok)
    out = torch.empty(len(want), V, dtype=torch.float32, device=self.device)
    if rows == 0:
      return out
    R = self._max_rows
    done_want = 0
    for lo in range(0, rows, R):
      hi = min(rows, lo + R)
      n = hi - lo
      w = [x - lo for x in want if lo <= x < hi]
      host = self._desc_host
      host[0:n] = torch.tensor(tok[lo:hi], dtype=torch.int32)
      host[R : R + n] = torch.tensor(grp[lo:hi], dtype=torch.int32)
      host[2 * R : 2 * R + n] = torch.tensor(pos[lo:hi], dtype=torch.int32)
      if w:
        host[3 * R : 3 * R + len(w)] = torch.tensor(w, dtype=torch.int32)
      # query tiles: every run of consecutive positions (an entry, cut at the slice) in pieces of at most 16 rows
      # and the runs themselves (recurrent mixers walk a run in order from its group's state)
      tiles, cuts = [], []
      for a, b in runs:
        a, b = max(a, lo), min(b, hi)
        if a < b:
          cuts.append(a - lo)
        tiles.extend(range(a - lo, b - lo, QUERY_TILE_ROWS))
      tiles.append(n)
      cuts.append(n)
      host[4 * R : 4 * R + len(tiles)] = torch.tensor(tiles, dtype=torch.int32)
      host[5 * R + 8 : 5 * R + 8 + len(cuts)] = torch.tensor(cuts, dtype=torch.int32)
      if lo:
        torch.cuda.current_stream(self.device).synchronize()  # the previous slice has read the staging buffer
      self._desc_dev.copy_(host, non_blocking=True)
      p = self._desc_dev.data_ptr()
      dst = out[done_want : done_want + len(w)]
      self._run(n, p, p + 4 * R, p + 8 * R, len(w), p + 12 * R, dst, len(tiles) - 1, p + 16 * R, n_runs=len(cuts) - 1, runs_ptr=p + 4 * (5 * R + 8))
      done_want += len(w)
    torch.cuda.current_stream(self.device).synchronize()  # the pinned staging buffer is free again when step returns
    return out

  def _sample(self, logits: torch.Tensor, rows: int, token_out: torch.Tensor, log_prob_out: Optional[torch.Tensor], row_offset: int) -> None:
    cfg = self.config
    _lib.check(self.lib.mtx_sample_rows(
        ctypes.c_void_p(logits.data_ptr()), rows, int(logits.stride(0)), int(cfg.vocab_size), _lib.SAMPLING[cfg.decode_sampling_strategy],
        int(cfg.decode_sampling_top_k), float(cfg.decode_sampling_nucleus_p), float(cfg.decode_sampling_temperature),
        ctypes.c_void_p(self._rng_state.data_ptr()), row_offset, ctypes.c_void_p(self._sample_scratch.data_ptr()),
        ctypes.c_void_p(token_out.data_ptr()), ctypes.c_void_p(log_prob_out.data_ptr()) if log_prob_out is not None else None, self._stream()))
    self._rng_state[0:1] += 1  # every draw has its own noise

  # -- the engine API -----------------------------------------------------------------------------

  def prefill(self, *, params: Any = None, padded_tokens: Any, true_length: int, existing_prefix: Any = None, images: Any = None,
              sampler: Any = None, rng: Any = None, request_id: Any = None, slot: Optional[int] = None, return_prompt_logp: bool = False):
    """maxengine.py:533-574 for one sequence; the rows go straight into the pages of `slot` (required).  `existing_prefix`
    (chunked prefill): the slot already holds that prefix and grows."""
    self._require_params(params)
    if slot is None:
      raise ValueError("a layered model prefills into the pages of a slot: pass slot=")
    if return_prompt_logp:
      raise NotImplementedError("return_prompt_logp is outside the decode path")
    self._seed(rng)
    slot, true_length = int(slot), int(true_length)
    toks = torch.as_tensor(padded_tokens).reshape(-1)
    if true_length < 1 or true_length > toks.numel():
      raise ValueError(f"true_length={true_length} for {toks.numel()} padded tokens")
    start = 0
    if existing_prefix is not None:
      start = int(torch.as_tensor(existing_prefix.common_prefix_tokens).reshape(-1).numel())
      if int(self.page_state.sequence_lengths[slot]) != start:
        raise ValueError(f"slot {slot} holds {int(self.page_state.sequence_lengths[slot])} tokens, the prefix has {start}")
    else:
      self.release_pages(slot)
    if start + true_length >= int(self.config.max_target_length):
      raise ValueError(f"{start + true_length} prompt tokens leave no room to decode (max_target_length={self.config.max_target_length})")
    logits = self.step([(slot, toks[:true_length].tolist(), [true_length - 1])])
    self._sample(logits, 1, self._first_token, self._first_log_prob if self.config.return_log_prob else None, 0x40000000)
    first = self._first_token.clone().reshape(1, 1)
    n = start + true_length
    prefix = {
        "logits": logits.reshape(1, 1, -1),
        "cache": {"slot": slot, "prefill_length": n},  # the keys and values are in the slot's pages already
        "next_pos": torch.full((1, 1), n, dtype=torch.int32, device=self.device),
        "generated_tokens": torch.zeros((1, 1), dtype=torch.int32, device=self.device),
        "tokens": first,
    }
    data = torch.cat((first, torch.ones_like(first), torch.zeros_like(first)), dim=1)
    lp = self._first_log_prob.clone().reshape(1, 1) if self.config.return_log_prob else None
    return prefix, ResultTokens(data=data, log_prob=lp)

  def insert(self, prefix: dict, decode_state: dict, slot: int, request_id: Any = None) -> dict:
    """maxengine.py:1166-1192.  The prefix lives in the pages of the slot it was prefilled into: that must be `slot`."""
    if decode_state is not self._state:
      raise ValueError("decode_state must be the dict returned by this engine's init_decode_state (it is donated)")
    slot = int(slot)
    if int(prefix["cache"]["slot"]) != slot:
      raise ValueError(f"this prefix was prefilled into slot {prefix['cache']['slot']}, not {slot}")
    self._next_pos[slot].copy_(prefix["next_pos"][0])
    self._generated[slot].copy_(prefix["generated_tokens"][0])
    self._tokens[slot].copy_(prefix["tokens"][0])
    self._active[slot].fill_(1)
    self._logits[slot].copy_(prefix["logits"][0])
    return decode_state

  def fill_synthetic_context(self, prefill_lengths, ar_lengths=None, seed: int = 7) -> dict:
    """Benchmark set-up (as MaxEngine.fill_synthetic_context): every slot holds a context of the given length without a prefill
    having run -- its pages are reserved, the pools hold random-normal rows, the recurrent states small random numbers."""
    B = self.max_concurrent_decodes
    state = self.init_decode_state()
    g = torch.Generator(device=self.device).manual_seed(seed)
    ps = self.page_state
    for slot in range(B):
      n = int(prefill_lengths[slot]) + (int(ar_lengths[slot]) if ar_lengths is not None else 0)
      ps = self.page_manager.extend_pages(ps, slot, n)
      if int(ps.sequence_lengths[slot]) != n:
        raise ValueError("pagedattn_num_pages is too small for the synthetic contexts")
      self._next_pos[slot].fill_(n)
    self.page_state = ps
    self._upload_page_map()
    for buf in self._pool_tensors:
      flat = buf.view(-1)
      for lo in range(0, flat.numel(), 1 << 26):
        n = min(1 << 26, flat.numel() - lo)
        flat[lo : lo + n] = torch.randn(n, device=self.device, generator=g).to(buf.dtype)
    for st in self._states:
      for t in st:
        t.copy_(torch.randn(t.shape, device=self.device, generator=g) * 0.1)
    self._active.fill_(1)
    self._tokens.copy_(torch.randint(0, int(self.config.vocab_size), self._tokens.shape, device=self.device, generator=g, dtype=torch.int32))
    return state

  def bulk_insert(self, prefix: dict, decode_state: dict, slots: list) -> dict:
    raise NotImplementedError("a paged prefix belongs to one slot")

  def _decode_rows(self) -> None:
    """One row per slot: token and position from the device state, the slot's pages grown by one token on the host."""
    B = self.max_concurrent_decodes
    ps = self.page_manager.update_decode_pages(self.page_state)
    grew = ps.has_active_page & (ps.num_pages_used * self.page_manager.tokens_per_page < ps.sequence_lengths)
    if grew.any():
      raise ValueError(f"the page pool is exhausted: slots {np.flatnonzero(grew).tolist()} cannot grow")
    self.page_state = ps
    self._upload_page_map()
    # rows of empty slots are parked in group B: they must not touch the state of a slot that was prefilled but not yet inserted
    torch.where(self._active.view(-1) != 0, self._slot_ids, torch.full_like(self._slot_ids, B), out=self._decode_groups)
    self._run(B, self._tokens.data_ptr(), self._decode_groups.data_ptr(), self._next_pos.data_ptr(), B, self._slot_ids.data_ptr(), self._logits,
              B, self._decode_tiles.data_ptr(), graph=self.use_cuda_graph, n_runs=B, runs_ptr=self._decode_tiles.data_ptr())
    self._sample(self._logits.view(B, -1), B, self._tokens, self._log_prob, 0)
    # bookkeeping of maxengine.py:913-928 for the occupied slots (empty ones stay at position 0 on page 0)
    self._next_pos.add_(self._active)
    self._generated.add_(self._active)
    self._result[:, 0:1].copy_(self._tokens)
    self._result[:, 1:2].copy_(self._active)
    self._result[:, 2:3].copy_(self._generated)

  def generate(self, params: Any, decode_state: dict, sampler: Any = None, rng: Any = None):
    if decode_state is not self._state:
      raise ValueError("decode_state must be the dict returned by this engine's init_decode_state (it is donated)")
    self._require_params(params)
    self._seed(rng)
    self._decode_rows()
    return decode_state, ResultTokens(data=self._result.clone(), log_prob=self._log_prob.clone() if self._log_prob is not None else None)

  def generate_to_host(self, params: Any, decode_state: dict, host_result: torch.Tensor, host_tokens: Optional[torch.Tensor] = None,
                       host_log_prob: Optional[torch.Tensor] = None, sync: bool = False):
    if decode_state is not self._state:
      raise ValueError("decode_state must be the dict returned by this engine's init_decode_state (it is donated)")
    self._require_params(params)
    if host_tokens is not None:
      self._tokens.copy_(host_tokens.reshape(self._tokens.shape), non_blocking=True)
    self._decode_rows()
    host_result.copy_(self._result, non_blocking=True)
    if host_log_prob is not None and self._log_prob is not None:
      host_log_prob.copy_(self._log_prob, non_blocking=True)
    if sync:
      torch.cuda.current_stream(self.device).synchronize()
    return decode_state, ResultTokens(data=host_result, log_prob=host_log_prob)
