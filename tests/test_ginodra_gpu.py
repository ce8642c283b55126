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
    "no_input_convolutions_at_all": lambda: {k: v for k, v in model([att(gi.dense_ff(24)), dlt()]).items() if k != "canon"},
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


def test_mechanism_functions_of_the_oracle_agree_with_closed_forms():
  # the oracle's own pieces against hand-computable cases (so a shared misreading cannot hide in both)
  x = np.array([[1.0, -1.0, 3.0, 4.0]])
  assert np.allclose(ref.group_norm(x, np.array([1.0, 2.0, 1.0, 1.0]), 2, 0.0), [[1.0, -2.0, 3.0 / np.sqrt(12.5), 4.0 / np.sqrt(12.5)]])
  h = np.array([[1.0], [10.0], [100.0]])
  assert ref.causal_conv(h, np.array([[3.0, 2.0, 1.0]])).ravel().tolist() == [1.0, 12.0, 123.0]  # the last tap is the row itself
  r = ref.rotate_half(np.array([[1.0, 5.0, 0.0, 0.0]]), np.array([2]), 100.0)  # pairs (0, 2) and (1, 3); angles 2 and 2 / 10
  assert np.allclose(r[0], [np.cos(2.0), 5 * np.cos(0.2), np.sin(2.0), 5 * np.sin(0.2)])
  assert np.allclose(ref.distance_slopes(4), [0.25, 0.0625, 0.015625, 0.00390625])
  p = ref.softmax_rows(np.zeros((2, 2)), np.array([[True, False], [True, True]]), sink=0.0)  # the sink counts once, like a key of score 0
  assert np.allclose(p, [[0.5, 0.0], [1 / 3, 1 / 3]])
  assert ref.window_mask(4, 2).astype(int).tolist() == [[1, 0, 0, 0], [1, 1, 0, 0], [0, 1, 1, 0], [0, 0, 1, 1]]
  # delta rule, two tokens along the same unit key e0: the second write first takes a2 of what the state holds along e0
  k = np.array([[2.0, 0.0], [2.0, 0.0]])
  o, S = ref.delta_scan(np.ones((2, 2)), k, np.array([[1.0], [0.0]]), np.full((2, 2), 0.5), np.array([[0.0, 0.0], [0.25, 0.0]]))
  u0 = 2.0 / np.sqrt(4.0 + 1e-6)
  assert np.isclose(o[0, 0], 2.0) and np.isclose(S[0, 0], 0.5 * 2.0 - 0.25 * u0 * u0 * 2.0)
  assert np.isclose(ref.squared_relu_ff(np.array([[1.0, -2.0]]), np.array([[3.0, 0.0], [0.0, 1.0]]), np.array([[1.0, 1.0]]))[0, 0], 9.0)


# ---- schedules: the logits of a position do not depend on how it got there --------------------------------------------------------

def test_prefill_equals_token_by_token_decoding():
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=1)
  toks = tokens_for(cfg, 45)
  want = ref.forward(cfg, t, toks)
  engine = make_engine(cfg, t)
  first = whole(engine, toks)
  assert rel_err(first, want) < TIGHT
  rows = [engine.step([(1, [tok], [0])]).cpu().numpy() for tok in toks]
  engine.release_pages(1)
  assert rel_err(np.concatenate(rows), want) < TIGHT
  assert rel_err(np.concatenate(rows), first) < 1e-5


@pytest.mark.parametrize("sizes", [[2, 2, 2, 3, 5, 16, 17, 15], [7, 1, 1, 2, 33, 18], [1, 61], [16, 16, 30], [31, 31]])
def test_portions_of_any_size(sizes):
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=2)
  toks = tokens_for(cfg, sum(sizes))
  want = ref.forward(cfg, t, toks)
  engine = make_engine(cfg, t, tokens_per_page=8)
  got, at = [], 0
  for n in sizes:
    got.append(engine.step([(2, toks[at : at + n], list(range(n)))]).cpu().numpy())
    at += n
  assert rel_err(np.concatenate(got), want) < TIGHT


@pytest.mark.parametrize("dtype,tol", [("float32", TIGHT), ("bfloat16", 3e-2)])
def test_a_step_longer_than_the_engine_takes_at_once_runs_in_slices(dtype, tol):
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=4)
  toks = {0: tokens_for(cfg, 50, seed=1), 1: tokens_for(cfg, 27, seed=2)}
  engine = make_engine(cfg, t, dtype=dtype, max_step_rows=19)  # slices cut both runs; the states and the convolutions' rings cross the cuts
  out = engine.step([(s, v, list(range(len(v)))) for s, v in toks.items()]).cpu().numpy()
  want = np.concatenate([ref.forward(cfg, t, v) for v in toks.values()])
  assert rms_err(out, want) < tol


def test_unequal_requests_in_one_batch_equal_each_alone_and_freed_slots_and_pages_are_reused():
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=3)
  lens = {"a": 43, "b": 9, "c": 1, "d": 14, "e": 37, "f": 6}
  toks = {k: tokens_for(cfg, n, seed=ord(k)) for k, n in lens.items()}
  want = {k: ref.forward(cfg, t, v) for k, v in toks.items()}
  # 19 usable pages of 4 tokens: a + b + c + d take 11 + 3 + 1 + 4; e and f only fit into pages that were given back, and they
  # inherit state slots whose recurrent state and convolution rings b and c left behind
  engine = make_engine(cfg, t, tokens_per_page=4, num_pages=20, max_len=64)
  got, at = {k: [] for k in toks}, {k: 0 for k in toks}
  slot_of = {"a": 0, "b": 1, "c": 2, "d": 3}
  plan = [
      [("a", 5), ("b", 2), ("c", 1), ("d", 3)],
      [("a", 1), ("b", 7), ("d", 1)],
      [("a", 19), ("d", 10)],
      [("a", 1), ("e", 4), ("f", 2)],
      [("a", 17), ("e", 1), ("f", 4)],
      [("e", 32)],
  ]
  for step in plan:
    for k, _ in step:
      if k not in slot_of:
        done = [r for r, s in slot_of.items() if at[r] == lens[r]]
        slot_of[k] = slot_of.pop(done[0])
    out = engine.step([(slot_of[k], toks[k][at[k] : at[k] + n], list(range(n))) for k, n in step]).cpu().numpy()
    for k, n in step:
      got[k].append(out[:n])
      out = out[n:]
      at[k] += n
      if at[k] == lens[k]:
        engine.release_pages(slot_of[k])
  for k in toks:
    assert at[k] == lens[k]
    assert rel_err(np.concatenate(got[k]), want[k]) < TIGHT, k


def test_a_reused_slot_starts_from_zero_state_even_without_a_release_clearing_it():
  cfg = model([dlt(gi.dense_ff(24)), att(), lat()], taps=4)
  t = ref.random_model(cfg, seed=8)
  engine = make_engine(cfg, t)
  a, b = tokens_for(cfg, 30, seed=1), tokens_for(cfg, 12, seed=2)
  engine.step([(0, a, [])])
  for st in engine._states:  # leave the first request's state and rings (and some dirt) behind when the slot is handed on
    for s in st:
      s[0].add_(3.0)
  ps = engine.page_manager.release_pages(page_state=engine.page_state, page_group_id=0)
  engine.page_state = ps
  assert rel_err(engine.step([(0, b, list(range(12)))]).cpu().numpy(), ref.forward(cfg, t, b)) < TIGHT


def test_pool_exhaustion_is_an_error_not_a_wrong_answer():
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=3)
  engine = make_engine(cfg, t, tokens_per_page=4, num_pages=5, max_len=64)
  engine.step([(0, tokens_for(cfg, 10), [9])])
  with pytest.raises(ValueError):
    engine.step([(1, tokens_for(cfg, 9), [8])])


def test_long_decoding_across_many_pages():
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=6)
  toks = tokens_for(cfg, 150)
  want = ref.forward(cfg, t, toks)
  engine = make_engine(cfg, t, tokens_per_page=4, num_pages=50)
  got = [engine.step([(3, toks[:5], list(range(5)))]).cpu().numpy()]
  got += [engine.step([(3, [tok], [0])]).cpu().numpy() for tok in toks[5:]]
  assert rel_err(np.concatenate(got), want) < TIGHT


# ---- far keys, window edges, sinks, page borders, the first tokens ------------------------------------------------------------------

def _peaky(cfg, seed, times=8.0):
  """Scores that spread widely, so that single keys (also far ones, also the one at a window's edge) carry most of a query's
  weight; slow decays and small removal rates, so that a token hundreds of steps back still matters in the recurrence."""
  t = ref.random_model(cfg, seed=seed)
  for i, l in enumerate(cfg["layers"]):
    p = f"l{i}.mix."
    if l["type"] == "attention":
      t[p + "q.norm"] = t[p + "q.norm"] * times
    elif l["type"] == "latent_attention":
      t[p + "uq"] = t[p + "uq"] * times
    else:
      t[p + "w0"] = t[p + "w0"] - 6.0
      t[p + "a.b"] = t[p + "a.b"] - 3.0
  return {k: ref.bf16_values(v) for k, v in t.items()}


@pytest.mark.parametrize("page", [4, 16, 64])
def test_far_keys_and_page_borders(page):
  cfg = model([lat(), dlt(), lat(gi.dense_ff(24))], softcap=0.0)
  t = _peaky(cfg, seed=21)
  n = 330
  toks = tokens_for(cfg, n)
  want = ref.forward(cfg, t, toks)
  assert rms_err(ref.forward(cfg, t, toks, fault={"horizon": 300})[301:], want[301:]) > 1e-3  # losing keys 300 back would show
  engine = make_engine(cfg, t, tokens_per_page=page, num_pages=700 // page + 2, max_len=400)
  assert rel_err(whole(engine, toks), want) < TIGHT
  # a prompt that ends at, one before and one after a page border, then decoding across the next borders
  for cut in (2 * page - 1, 2 * page, 2 * page + 1):
    got = [engine.step([(1, toks[:cut], list(range(cut)))]).cpu().numpy()]
    got += [engine.step([(1, [tok], [0])]).cpu().numpy() for tok in toks[cut : cut + page + 3]]
    engine.release_pages(1)
    assert rel_err(np.concatenate(got), want[: cut + page + 3]) < TIGHT, cut
  # far keys seen from decoded tokens
  got = [engine.step([(2, toks[:310], [])]).cpu().numpy()] + [engine.step([(2, [tok], [0])]).cpu().numpy() for tok in toks[310:]]
  assert rel_err(np.concatenate(got[1:]), want[310:]) < TIGHT


@pytest.mark.parametrize("dtype,tol", [("float32", TIGHT), ("bfloat16", 3e-2)])
@pytest.mark.parametrize("window", [1, 7, 16, 33])
def test_keys_just_inside_and_just_outside_the_window(window, dtype, tol):
  """Peaky scores: a query's weight sits on few keys, often the oldest one it may see.  The oracle with a window one key wider
  gives clearly different logits, so a window that is one token off would show; the engine agrees with the exact one over a
  whole prompt, over portions that end around the window's edge, and decoding one token at a time."""
  cfg = model([att(window=window, heads=4, kv_heads=2, dim=16, vdim=16), att(gi.dense_ff(24), window=window + 2, kv_from=0, heads=4, kv_heads=2, dim=16, vdim=16)],
              softcap=0.0)
  t = _peaky(cfg, seed=30 + window, times=12.0)
  n = 3 * window + 40
  toks = tokens_for(cfg, n, seed=window)
  want = ref.forward(cfg, t, toks)
  for shift in (1, -1) if window > 1 else (1,):
    assert rms_err(ref.forward(cfg, t, toks, fault={"window_shift": shift})[window:], want[window:]) > 1.5 * 3e-2
  engine = make_engine(cfg, t, dtype=dtype, tokens_per_page=8, num_pages=40)
  err = rel_err if dtype == "float32" else rms_err
  assert err(whole(engine, toks), want) < tol
  for cuts in ([window - 1, 1, 1, window, 2], [window, window + 1, window - 1], [window + 1, 2, 2 * window - 3]):
    cuts = [c for c in cuts if c > 0]
    got, at = [], 0
    for c in cuts:
      got.append(engine.step([(1, toks[at : at + c], list(range(c)))]).cpu().numpy())
      at += c
    got += [engine.step([(1, [tok], [0])]).cpu().numpy() for tok in toks[at : at + window + 3]]
    engine.release_pages(1)
    assert err(np.concatenate(got), want[: at + window + 3]) < tol, cuts


@pytest.mark.parametrize("dtype,tol", [("float32", TIGHT), ("bfloat16", 3e-2)])
def test_a_sink_that_outweighs_the_keys(dtype, tol):
  cfg = model([lat(), lat(gi.dense_ff(24), heads=8, dim=16, rot_dim=16, vdim=16, kv_rank=48)], softcap=0.0)
  t = ref.random_model(cfg, seed=40)
  for i in range(2):
    t[f"l{i}.mix.sink"] = ref.bf16_values(t[f"l{i}.mix.sink"] + 3.0)
  toks = tokens_for(cfg, 70)
  want = ref.forward(cfg, t, toks)
  assert rms_err(ref.forward(cfg, t, toks, fault={"no_sink": True}), want) > 0.05  # leaving the sink out would show
  engine = make_engine(cfg, t, dtype=dtype, tokens_per_page=16, num_pages=20)
  err = rel_err if dtype == "float32" else rms_err
  assert err(whole(engine, toks), want) < tol
  got = [engine.step([(1, toks[:50], list(range(50)))]).cpu().numpy()] + [engine.step([(1, [tok], [0])]).cpu().numpy() for tok in toks[50:]]
  assert err(np.concatenate(got), want) < tol


def test_first_tokens_of_a_sequence():
  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=9)
  engine = make_engine(cfg, t)
  for n in (1, 2, 3, 4):
    toks = tokens_for(cfg, n, seed=n)
    assert rel_err(whole(engine, toks), ref.forward(cfg, t, toks)) < TIGHT
    got = [engine.step([(1, [tok], [0])]).cpu().numpy() for tok in toks]  # the rows before the start are zeros, not the ring's old rows
    engine.release_pages(1)
    assert rel_err(np.concatenate(got), ref.forward(cfg, t, toks)) < TIGHT


# ---- other sizes ------------------------------------------------------------------------------------------------------------------

SIZES = {
    "odd_width": lambda: model([att(gi.dense_ff(30)), dlt(gi.dense_ff(18)), lat()], width=36, vocab=47, groups=3),
    "heads_with_kv_heads_of_their_own": lambda: model([att(kv_heads=4)]),
    "one_head_everywhere": lambda: model([att(heads=1, kv_heads=1), dlt(heads=1), lat(heads=1)]),
    "value_size_over_key_size": lambda: model([att(dim=8, vdim=40), lat(dim=8, vdim=36)]),
    "latent_wider_than_the_heads": lambda: model([lat(heads=2, dim=8, rot_dim=4, vdim=8, q_rank=40, kv_rank=72)]),
    "rotated_part_of_two_channels": lambda: model([lat(rot_dim=2)]),
    "delta_heads_not_a_multiple_of_four": lambda: model([dlt(heads=2, dim=18)]),
    "wide_delta_heads": lambda: model([dlt(heads=2, dim=136)], width=64),
    "widest_delta_heads": lambda: model([dlt(heads=1, dim=256)], width=64),
    "shared_cache_two_layers_back": lambda: model([att(gi.dense_ff(24)), dlt(), att(kv_from=0, window=30), att(kv_from=0, window=2)]),
    "two_taps": lambda: model([att(gi.dense_ff(24)), dlt(gi.dense_ff(24)), lat(gi.dense_ff(24))], taps=2),
    "seven_taps": lambda: model([att(gi.dense_ff(24)), dlt(gi.dense_ff(24)), lat(gi.dense_ff(24))], taps=7),
    "more_taps_than_the_convolution_keeps_a_table_for": lambda: model([att(gi.dense_ff(24)), dlt(gi.dense_ff(24))], taps=20),
    "layers_without_feed_forward": lambda: model([att(), dlt(), lat()]),
    "ten_norm_groups": lambda: model([att(gi.dense_ff(24)), dlt()], groups=10),  # (groups of one or two channels make x / sqrt(x^2 + eps) ill-conditioned near 0)
    "eight_norm_groups": lambda: model([att(gi.dense_ff(24)), dlt()], groups=8),
    "five_norm_groups": lambda: model([att(gi.dense_ff(24)), dlt()], groups=5),
}


@pytest.mark.parametrize("case", sorted(SIZES))
def test_other_sizes(case):
  cfg = SIZES[case]()
  t = ref.random_model(cfg, seed=13)
  toks = tokens_for(cfg, 41)
  want = ref.forward(cfg, t, toks)
  engine = make_engine(cfg, t, tokens_per_page=8)
  got = [engine.step([(0, toks[:22], list(range(22)))]).cpu().numpy(), engine.step([(0, toks[22:39], list(range(17)))]).cpu().numpy()]
  got += [engine.step([(0, [tok], [0])]).cpu().numpy() for tok in toks[39:]]
  assert rel_err(np.concatenate(got), want) < TIGHT


@pytest.mark.parametrize("case", sorted(SIZES))
def test_other_sizes_on_a_bfloat16_engine(case):
  # (odd widths and sizes take the unvectorised loads of the tensor-core projections and the row kernel of the attention)
  cfg = SIZES[case]()
  t = ref.random_model(cfg, seed=14)
  toks = tokens_for(cfg, 41)
  want = ref.forward(cfg, t, toks)
  engine = make_engine(cfg, t, dtype="bfloat16", tokens_per_page=8)
  got = [engine.step([(0, toks[:22], list(range(22)))]).cpu().numpy(), engine.step([(0, toks[22:39], list(range(17)))]).cpu().numpy()]
  got += [engine.step([(0, [tok], [0])]).cpu().numpy() for tok in toks[39:]]
  assert rms_err(np.concatenate(got), want) < 3e-2


@pytest.mark.parametrize("case", ["default", "tiles"])
def test_bfloat16_engine_is_within_rounding_of_the_exact_model(case):
  if case == "default":
    cfg = DEFAULT()
  else:  # sizes made of whole tiles of the tensor-core kernels
    cfg = model([dlt(gi.dense_ff(128), heads=2, dim=64), att(gi.dense_ff(128), heads=4, kv_heads=2, dim=64, vdim=64, window=40),
                 att(gi.dense_ff(64), heads=4, kv_heads=2, dim=64, vdim=64, window=24, kv_from=1),
                 lat(gi.dense_ff(128), heads=4, dim=32, rot_dim=32, vdim=32, q_rank=64, kv_rank=96)], width=128, vocab=256)
  t = ref.random_model(cfg, seed=15)
  toks = tokens_for(cfg, 90)
  want = ref.forward(cfg, t, toks)
  engine = make_engine(cfg, t, dtype="bfloat16", tokens_per_page=16, num_pages=30)
  assert rms_err(whole(engine, toks), want) < 3e-2
  got = [engine.step([(1, toks[:70], list(range(70)))]).cpu().numpy()] + [engine.step([(1, [tok], [0])]).cpu().numpy() for tok in toks[70:]]
  assert rms_err(np.concatenate(got), want) < 3e-2


# ---- the tensor-core attention with the optional parts (bf16, head sizes in multiples of 16) ----------------------------------------

@pytest.mark.parametrize("kind,heads,kv_heads,dim,page", [("att", 4, 2, 64, 16), ("att", 2, 2, 16, 8), ("att", 8, 1, 32, 64), ("att", 6, 2, 48, 4),
                                                          ("lat", 8, 1, 64, 16), ("lat", 3, 1, 128, 32), ("lat_narrow_ff", 12, 1, 128, 16), ("lat", 16, 1, 96, 16), ("lat", 2, 1, 256, 16)])
def test_tensor_core_attention_shapes_and_schedules(kind, heads, kv_heads, dim, page):
  """Head sizes of the tensor-core arm with slopes and a window (attention) or a sink and one key head (latent attention, `dim`
  = latent + rotated part), prompts in portions that end inside, at and after the 64-key tiles, 16-row query tiles that start
  anywhere, then single tokens; peaky scores so that single far keys matter."""
  if kind == "att":
    layers = [att(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, window=70), att(gi.dense_ff(32), heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, window=0)]
  elif kind == "lat_narrow_ff":  # (the key splits' partial results are wider than any activation of the model)
    layers = [lat(gi.dense_ff(16), heads=heads, dim=8, rot_dim=dim // 4, vdim=8, q_rank=24, kv_rank=dim - dim // 4)]
  else:
    layers = [lat(heads=heads, dim=16, rot_dim=dim // 4, vdim=24, q_rank=24, kv_rank=dim - dim // 4), dlt(gi.dense_ff(32), heads=2, dim=16)]
  cfg = model(layers, width=64, vocab=90, softcap=0.0)
  t = _peaky(cfg, seed=dim + heads, times=6.0)
  n = 150
  toks = tokens_for(cfg, n, seed=dim)
  want = ref.forward(cfg, t, toks)
  engine = make_engine(cfg, t, dtype="bfloat16", tokens_per_page=page, num_pages=2 * (n // page + 2) + 2, max_len=n + 8)
  assert rms_err(whole(engine, toks), want) < 3e-2
  for cuts in ([63, 1, 1, 30, 33], [64, 64], [65, 5, 58, 9], [31, 2, 31, 33, 7, 25]):
    got, at = [], 0
    for c in cuts:
      got.append(engine.step([(1, toks[at : at + c], list(range(c)))]).cpu().numpy())
      at += c
    got += [engine.step([(1, [tok], [0])]).cpu().numpy() for tok in toks[at : at + 6]]
    engine.release_pages(1)
    assert rms_err(np.concatenate(got), want[: at + 6]) < 3e-2, cuts
  # two sequences side by side, one in the middle of its prompt, one decoding
  engine.step([(0, toks[:70], []), (2, toks[:101], [])])
  out = engine.step([(0, toks[70:90], list(range(20))), (2, [toks[101]], [0])]).cpu().numpy()
  assert rms_err(out, np.concatenate([want[70:90], want[101:102]])) < 3e-2


# ---- the framework's entry point: scheduler, sampler -------------------------------------------------------------------------------

def test_greedy_generation_through_the_offline_engine():
  from maxtext_indextts2_b200 import offline_engine

  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=17)
  config = pyconfig.from_model_dict(cfg, dtype="float32", per_device_batch_size=2, max_target_length=64, pagedattn_tokens_per_page=4,
                                    pagedattn_num_pages=30, decode_sampling_strategy="greedy")
  eng = offline_engine.OfflineEngine(config, params=as_torch(t))
  prompts = [tokens_for(cfg, n, seed=30 + n) for n in (5, 11, 3, 8, 2)]  # five prompts over two slots: slots, pages and state are reused
  outs = eng.batch_inference(prompts, max_decode_length=9)
  for prompt, out in zip(prompts, outs):
    seq = list(prompt)
    for _ in range(9):
      logits = ref.forward(cfg, t, seq)[-1]
      top2 = np.sort(logits)[-2:]
      assert float(top2[1] - top2[0]) > 1e-4, "near-tie in the test's own model; change the seed"
      seq.append(int(logits.argmax()))
    assert out.token_ids.tolist() == seq[len(prompt):]


# ---- the command lines: prompts in, tokens out; a trace of batched steps replayed through bin/trace_run --------------------------------

def _write_model_dir(path, cfg, t):
  import json
  import os

  from tests.test_gugidra_host import _write_safetensors

  os.makedirs(path)
  with open(path / "config.json", "w") as f:
    json.dump(cfg, f)
  _write_safetensors(path / "model.safetensors", as_torch(t))


def test_decode_command_line_generates_the_oracles_greedy_tokens(tmp_path):
  import json
  import os
  import subprocess
  import sys

  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=19)
  _write_model_dir(tmp_path / "model", cfg, t)
  prompts = [tokens_for(cfg, n, seed=50 + n) for n in (7, 3)]
  root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
  cmd = [sys.executable, "-m", "maxtext_indextts2_b200.decode", f"model_dir={tmp_path / 'model'}", "dtype=float32", "decode_sampling_strategy=greedy",
         "pagedattn_tokens_per_page=8", "--max-decode", "6"]
  for p in prompts:
    cmd += ["--prompt", ",".join(str(x) for x in p)]
  r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=root)
  assert r.returncode == 0, r.stderr[-2000:]
  outs = {d["prompt"]: d["tokens"] for d in (json.loads(l) for l in r.stdout.splitlines() if l.startswith("{"))}
  for i, prompt in enumerate(prompts):
    seq = list(prompt)
    for _ in range(6):
      logits = ref.forward(cfg, t, seq)[-1]
      top2 = np.sort(logits)[-2:]
      assert float(top2[1] - top2[0]) > 1e-4, "near-tie in the test's own model; change the seed"
      seq.append(int(logits.argmax()))
    assert outs[i] == seq[len(prompt):]


@pytest.mark.parametrize("dtype,tol", [("float32", TIGHT), ("bfloat16", 5e-2)])  # (bfloat16: per step, some of few rows)
def test_trace_runner_replays_a_mixed_schedule(tmp_path, dtype, tol):
  import json
  import os
  import subprocess

  cfg = DEFAULT()
  t = ref.random_model(cfg, seed=23)
  model_dir = tmp_path / "model"
  _write_model_dir(model_dir, cfg, t)
  lens = {"a": 70, "b": 9, "c": 33, "d": 5, "e": 40, "f": 20}
  toks = {k: tokens_for(cfg, n, seed=ord(k)) for k, n in lens.items()}
  # four pages of 64 tokens: a, b, c fill them (2 + 1 + 1); d, e and f fit only into what b and c give back, and take their slots
  plan = [[("a", 30), ("b", 2)], [("a", 1), ("b", 7), ("c", 33)], [("a", 35), ("d", 2)], [("a", 1), ("d", 3), ("e", 39)], [("a", 3), ("e", 1), ("f", 20)]]
  at = {k: 0 for k in toks}
  lines, rows = [], []
  for n, step in enumerate(plan):
    entries, end = [], []
    for k, c in step:
      entries.append({"id": k, "tokens": toks[k][at[k] : at[k] + c], "want": list(range(c))})
      rows.append((n, k, at[k], c))
      at[k] += c
      if at[k] == lens[k]:
        end.append(k)
    lines.append(json.dumps({"step": n, "entries": entries, "end": end}))
  root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
  out_dir = tmp_path / "out"
  p = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(model_dir), "--dtype", dtype, "--out", str(out_dir), "--max-tokens", "256"],
                     input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
  assert p.returncode == 0, p.stderr[-2000:]
  assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {n}" for n in range(len(plan))]
  want = {k: ref.forward(cfg, t, v) for k, v in toks.items()}
  V = cfg["vocab"]
  errs = []
  for n in range(len(plan)):
    got = np.fromfile(out_dir / f"{n}.f32", dtype="<f4").reshape(-1, V)
    exp = np.concatenate([want[k][lo : lo + c] for s, k, lo, c in rows if s == n])
    assert got.shape == exp.shape
    errs.append(rms_err(got, exp))
  assert max(errs) < tol, errs
