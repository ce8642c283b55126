"""The Ginodra design on the layered engine against the plain restatement in oracle/ginodra_ref.py (numpy float64, same weights).

Small configurations with random weights; where random weights would hide a fault (a far key among hundreds, a sink, a window's
edge, a state that is lost or not reset) the weights are made so that it shows.  float32 engines are compared tightly, bfloat16
ones within rounding.
"""

import numpy as np
import pytest
import torch

from maxtext_indextts2_b200 import ginodra as gi
from maxtext_indextts2_b200 import maxengine, pyconfig
from oracle import ginodra_ref as ref

pytestmark = pytest.mark.gpu

TIGHT = 3e-5


def as_torch(t):
  return {k: torch.from_numpy(np.asarray(v)).to(torch.bfloat16) for k, v in t.items()}


def make_engine(cfg_dict, tensors, dtype="float32", slots=4, tokens_per_page=4, num_pages=60, max_len=200, **kw):
  config = pyconfig.from_model_dict(cfg_dict, dtype=dtype, per_device_batch_size=slots, max_target_length=max_len,
                                    pagedattn_tokens_per_page=tokens_per_page, pagedattn_num_pages=num_pages, **kw)
  engine = maxengine.MaxEngine(config)
  engine.load_params(as_torch(tensors))
  engine.init_decode_state()
  return engine


def tokens_for(cfg_dict, n, seed=5):
  return np.random.Generator(np.random.PCG64(seed)).integers(0, cfg_dict["vocab"], size=n).tolist()


def rel_err(got, want):
  got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
  return float(np.abs(got - want).max() / np.abs(want).max())


def rms_err(got, want):
  got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
  return float(np.sqrt(((got - want) ** 2).mean()) / np.sqrt((want**2).mean()))


def whole(engine, toks, slot=0):
  out = engine.step([(slot, toks, list(range(len(toks))))]).cpu().numpy()
  engine.release_pages(slot)
  return out


def att(mlp=None, **kw):
  args = dict(heads=4, kv_heads=2, dim=24, vdim=20, window=9, scale=0.31)
  args.update(kw)
  return gi.attention_layer(mlp=mlp, **args)


def lat(mlp=None, **kw):
  args = dict(heads=3, dim=12, rot_dim=8, vdim=20, q_rank=10, kv_rank=28, rot_base=100.0, scale=0.27)
  args.update(kw)
  return gi.latent_layer(mlp=mlp, **args)


def dlt(mlp=None, **kw):
  args = dict(heads=3, dim=12)
  args.update(kw)
  return gi.delta_layer(mlp=mlp, **args)


def model(layers, width=40, vocab=61, groups=2, taps=3, mult=0.4, scale=0.7, softcap=4.0):
  return gi.model_dict(width, vocab, layers, eps=1e-5, groups=groups, taps=taps, residual_mult=mult, logit_scale=scale, logit_softcap=softcap)


DEFAULT = lambda: model([dlt(gi.dense_ff(56)), att(gi.dense_ff(32)), att(gi.dense_ff(24), kv_from=1, window=5, scale=0.2), lat(gi.dense_ff(48))])

# ---- each mechanism alone ------------------------------------------------------------------------------------------------------

CASES = {
    "window_attention": lambda: model([att()]),
    "attention_no_window": lambda: model([att(window=0)]),
    "attention_one_kv_head": lambda: model([att(kv_heads=1)]),
    "attention_window_one": lambda: model([att(window=1)]),
    "shared_keys_and_values": lambda: model([att(), att(kv_from=0, window=4, scale=0.5)]),
    "latent_attention": lambda: model([lat()]),
    "latent_attention_one_head": lambda: model([lat(heads=1)]),
    "delta_rule": lambda: model([dlt()]),
    "delta_rule_one_head": lambda: model([dlt(heads=1, dim=20)]),
    "feed_forward": lambda: model([dlt(gi.dense_ff(56))]),
    "no_conv_taps": lambda: model([att(gi.dense_ff(24))], taps=1),
    "five_taps": lambda: model([att(gi.dense_ff(24)), dlt(gi.dense_ff(24))], taps=5),
    "one_norm_group": lambda: model([att(gi.dense_ff(24))], groups=1),
    "ten_norm_groups": lambda: model([lat(gi.dense_ff(24))], groups=10),
    "no_softcap_unit_scales": lambda: model([att(gi.dense_ff(24))], mult=1.0, scale=1.0, softcap=0.0),
    "all_mixers": DEFAULT,
}


@pytest.mark.parametrize("case", sorted(CASES))
def test_each_mechanism_alone(case):
  cfg = CASES[case]()
  t = ref.random_model(cfg, seed=11)
  toks = tokens_for(cfg, 37)
  want = ref.forward(cfg, t, toks)
  engine = make_engine(cfg, t)
  assert rel_err(whole(engine, toks), want) < TIGHT


@pytest.mark.parametrize("case", ["all_mixers", "latent_attention", "window_attention", "delta_rule"])
def test_bfloat16_engine_within_rounding(case):
  cfg = CASES[case]()
  t = ref.random_model(cfg, seed=3)
  toks = tokens_for(cfg, 41)
  want = ref.forward(cfg, t, toks)
  engine = make_engine(cfg, t, dtype="bfloat16")
  assert rms_err(whole(engine, toks), want) < 3e-2
