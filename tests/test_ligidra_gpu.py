"""The Ligidra design on the layered engine against the plain restatement in oracle/ligidra_ref.py (numpy float64, same weights).

Small configurations with random weights; where random weights would hide a fault (a far key among hundreds, a sink, a window's or
a pooled block's edge, a state that is lost or not reset) the weights are made so that it shows, and the oracle is told to make
that fault to prove it.  float32 engines are compared tightly, bfloat16 ones within rounding.
"""

import numpy as np
import pytest
import torch

from maxtext_indextts2_b200 import ligidra as lg
from maxtext_indextts2_b200 import maxengine, pyconfig
from oracle import ligidra_ref as ref

pytestmark = pytest.mark.gpu

TIGHT = 3e-5
LOOSE = 3e-2


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


def in_portions(engine, toks, cuts, slot=1, decode=0):
  """The sequence fed in portions of `cuts` tokens, then `decode` tokens one by one; every position's logits."""
  got, at = [], 0
  for c in cuts:
    got.append(engine.step([(slot, toks[at : at + c], list(range(c)))]).cpu().numpy())
    at += c
  got += [engine.step([(slot, [tok], [0])]).cpu().numpy() for tok in toks[at : at + decode]]
  engine.release_pages(slot)
  return np.concatenate(got)


SCALING = {"factor": 3.0, "low": 1.0, "high": 3.0, "original": 40}


def att(mlp=None, **kw):
  args = dict(heads=4, kv_heads=2, dim=12, vdim=20, window=9, pool=3, scale=0.31, softcap=6.0, rot_dims=8, rot_base=50.0, rot_scaling=SCALING)
  args.update(kw)
  return lg.attention_layer(mlp=mlp, **args)


def dlt(mlp=None, **kw):
  args = dict(heads=4, kv_heads=2, dim=12, vdim=10, taps=3)
  args.update(kw)
  return lg.delta_layer(mlp=mlp, **args)


def cdl(mlp=None, **kw):
  return dlt(mlp, per_channel=True, **kw)


def moe(experts=5, top=2, ff=14, shared_ff=10):
  return lg.moe_ff(experts, top, ff, shared_ff)


def model(layers, width=40, vocab=61, side_dim=6):
  return lg.model_dict(width, vocab, layers, eps=1e-5, side_dim=side_dim)


def weights(cfg, seed, toks=None):
  """Random weights; of eight seeds the one whose routers make the least close call on `toks` (no test rests on which of two
  nearly equal experts is chosen)."""
  if toks is None or not any(l.get("mlp") for l in cfg["layers"]):
    return ref.random_model(cfg, seed=seed)
  models = [ref.random_model(cfg, seed=s) for s in range(seed, seed + 8)]
  return max(models, key=lambda t: ref.closest_router_gap(cfg, t, toks))


DEFAULT = lambda: model([att(moe()), dlt(moe(4, 1, 12, 0)), att(moe(), kv_from=0, window=5, pool=2, scale=0.2), cdl(moe(6, 3, 10, 8))])

# ---- each mechanism alone ------------------------------------------------------------------------------------------------------

CASES = {
    "pooled_window_attention": lambda: model([att()], side_dim=0),
    "window_without_pooled_blocks": lambda: model([att(pool=0)], side_dim=0),
    "attention_without_window": lambda: model([att(window=0, pool=0)], side_dim=0),
    "attention_without_cap_scaling_rotation": lambda: model([att(softcap=0.0, rot_scaling=None), att(rot_dims=0)], side_dim=0),
    "attention_one_kv_head": lambda: model([att(kv_heads=1)], side_dim=0),
    "window_one_pool_one": lambda: model([att(window=1, pool=1)], side_dim=0),
    "shared_keys_and_values_other_window_and_blocks": lambda: model([att(), att(kv_from=0, window=4, pool=5, scale=0.5)], side_dim=0),
    "shared_keys_and_values_same_blocks": lambda: model([att(), att(kv_from=0, window=6, pool=3)], side_dim=0),
    "delta_rule": lambda: model([dlt()], side_dim=0),
    "delta_rule_heads_with_keys_of_their_own": lambda: model([dlt(kv_heads=4)], side_dim=0),
    "channel_delta_rule": lambda: model([cdl()], side_dim=0),
    "one_tap": lambda: model([dlt(taps=1), cdl(taps=1)], side_dim=0),
    "routed_feed_forward": lambda: model([dlt(moe())], side_dim=0),
    "routed_feed_forward_without_shared_expert_every_expert_chosen": lambda: model([dlt(moe(3, 3, 12, 0))], side_dim=0),
    "side_input": lambda: model([dlt(), att()], side_dim=5),
    "all_mixers": DEFAULT,
}


@pytest.mark.parametrize("case", sorted(CASES))
def test_each_mechanism_alone(case):
  cfg = CASES[case]()
  toks = tokens_for(cfg, 37)
  t = weights(cfg, 11, toks)
  want = ref.forward(cfg, t, toks)
  engine = make_engine(cfg, t)
  assert rel_err(whole(engine, toks), want) < TIGHT


@pytest.mark.parametrize("case", ["all_mixers", "pooled_window_attention", "delta_rule", "channel_delta_rule", "side_input"])
def test_bfloat16_engine_within_rounding(case):
  cfg = CASES[case]()
  toks = tokens_for(cfg, 41)
  t = weights(cfg, 3, toks)
  want = ref.forward(cfg, t, toks)
  engine = make_engine(cfg, t, dtype="bfloat16")
  assert rms_err(whole(engine, toks), want) < LOOSE


def test_mechanism_functions_of_the_oracle_agree_with_closed_forms():
  # the oracle's own pieces against hand-computable cases (so a shared misreading cannot hide in both)
  h = np.array([[1.0, 2.0], [3.0, 6.0]])
  assert np.allclose(ref.token_shift(h, np.array([0.5, 1.0])), [[0.5, 0.0], [2.0, 2.0]])  # the first row moves towards zero
  x = np.array([[10.0], [100.0], [1000.0]])
  assert ref.short_conv(x, np.array([[3.0, 2.0, 1.0]])).ravel().tolist() == [10.0, 120.0, 1230.0]  # the last tap is the row itself
  assert ref.visible(9, 4, 3) == ([6, 7, 8, 9], [0, 1])     # block 1 = 3..5 ends at 9 - 4
  assert ref.visible(8, 4, 3) == ([5, 6, 7, 8], [0])        # token 4 is neither in the window nor in a block that is complete before it
  assert ref.visible(3, 4, 3) == ([0, 1, 2, 3], [])
  assert ref.visible(5, 0, 3) == ([0, 1, 2, 3, 4, 5], [])
  r = ref.rotate_pairs(np.array([[[1.0, 0.0, 5.0, 7.0]]]), np.array([2]), np.array([0.25]))  # one pair turns by 0.5, the rest passes
  assert np.allclose(r[0, 0], [np.cos(0.5), np.sin(0.5), 5.0, 7.0])
  # one query, two keys of score 0 and a sink of 0: each key weighs 1 / 3
  o = ref.pooled_window_attention(np.zeros((2, 1, 2)), np.zeros((2, 1, 2)), np.array([[[3.0]], [[6.0]]]), 1.0, 0.0, 0, 0, np.array([0.0]))
  assert np.allclose(o[:, 0, 0], [1.5, 3.0])
  # gated delta rule: writing twice along the same unit key with beta = 1 replaces the value; the decay acts before the write
  k = np.array([[1.0, 0.0], [1.0, 0.0]])
  o, S = ref.gated_delta_scan(k, k, np.array([[2.0], [5.0]]), np.array([[1.0, 1.0], [0.5, 0.5]]), np.array([1.0, 1.0]))
  assert np.allclose(o[:, 0], [2.0, 5.0]) and np.isclose(S[0, 0], 5.0)
  o, S = ref.gated_delta_scan(k, k, np.array([[2.0], [5.0]]), np.array([[1.0, 1.0], [0.5, 0.5]]), np.array([1.0, 0.5]))
  assert np.isclose(S[0, 0], 1.0 + 0.5 * (5.0 - 1.0))
  c, w = ref.route(np.log(np.array([[1.0, 4.0, 3.0, 2.0]])), 2)
  assert c.tolist() == [[1, 2]] and np.allclose(w, [[0.4, 0.3]])  # the scores as they are, not renormalised


def test_scaled_frequencies_three_regimes():
  sc = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 8.0}
  f = ref.scaled_frequencies(6, 1000.0, sc)  # plain: 1, 0.1, 0.01 -> wavelengths 6.3, 63, 628; borders at 2 and 8
  s = (8.0 / (2 * np.pi) - 1.0) / 3.0
  assert np.allclose(f, [(1 - s) / 4.0 + s, 0.1 / 4.0, 0.01 / 4.0])
  assert np.allclose(ref.scaled_frequencies(2, 10.0, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64.0}), [1.0])  # short wavelength: kept
  assert np.allclose(lg.scaled_rot_frequencies(6, 1000.0, sc).numpy(), f)


# ---- schedules: the logits of a position do not depend on how it got there --------------------------------------------------------

def test_prefill_equals_token_by_token_decoding():
  cfg = DEFAULT()
  toks = tokens_for(cfg, 45)
  t = weights(cfg, 1, toks)
  want = ref.forward(cfg, t, toks)
  engine = make_engine(cfg, t)
  first = whole(engine, toks)
  assert rel_err(first, want) < TIGHT
  rows = in_portions(engine, toks, [], decode=len(toks))
  assert rel_err(rows, want) < TIGHT
  assert rel_err(rows, first) < 1e-5


@pytest.mark.parametrize("sizes", [[2, 2, 2, 3, 5, 16, 17, 15], [7, 1, 1, 2, 33, 18], [1, 61], [16, 16, 30], [31, 31]])
def test_portions_of_any_size(sizes):
  cfg = DEFAULT()
  toks = tokens_for(cfg, sum(sizes))
  t = weights(cfg, 2, toks)
  want = ref.forward(cfg, t, toks)
  engine = make_engine(cfg, t, tokens_per_page=8)
  assert rel_err(in_portions(engine, toks, sizes, slot=2), want) < TIGHT


@pytest.mark.parametrize("dtype,tol", [("float32", TIGHT), ("bfloat16", LOOSE)])
def test_a_step_longer_than_the_engine_takes_at_once_runs_in_slices(dtype, tol):
  cfg = DEFAULT()
  toks = {0: tokens_for(cfg, 50, seed=1), 1: tokens_for(cfg, 27, seed=2)}
  t = weights(cfg, 4, toks[0] + toks[1])
  engine = make_engine(cfg, t, dtype=dtype, max_step_rows=19)  # slices cut both runs; states, rings and pooled blocks cross the cuts
  out = engine.step([(s, v, list(range(len(v)))) for s, v in toks.items()]).cpu().numpy()
  want = np.concatenate([ref.forward(cfg, t, v) for v in toks.values()])
  assert rms_err(out, want) < tol


def test_unequal_requests_in_one_batch_equal_each_alone_and_freed_slots_and_pages_are_reused():
  cfg = DEFAULT()
  lens = {"a": 43, "b": 9, "c": 1, "d": 14, "e": 37, "f": 6}
  toks = {k: tokens_for(cfg, n, seed=ord(k)) for k, n in lens.items()}
  t = weights(cfg, 3, sum(toks.values(), []))
  want = {k: ref.forward(cfg, t, v) for k, v in toks.items()}
  # 19 usable pages of 4 tokens: a + b + c + d take 11 + 3 + 1 + 4; e and f only fit into pages that were given back, and they
  # inherit state slots whose recurrent state, rings and pooled blocks b and c left behind
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
  cfg = model([dlt(moe()), att(), cdl()])
  a, b = tokens_for(cfg, 30, seed=1), tokens_for(cfg, 12, seed=2)
  t = weights(cfg, 8, a + b)
  engine = make_engine(cfg, t)
  engine.step([(0, a, [])])
  for st in engine._states:  # leave the first request's state and rings (and some dirt) behind when the slot is handed on
    for s in st:
      s[0].add_(3.0)
  for pools in engine._pooled.values():  # ... and its pooled blocks
    for pool in pools:
      pool.add_(1.0)
  ps = engine.page_manager.release_pages(page_state=engine.page_state, page_group_id=0)
  engine.page_state = ps
  assert rel_err(engine.step([(0, b, list(range(12)))]).cpu().numpy(), ref.forward(cfg, t, b)) < TIGHT


def test_pool_exhaustion_is_an_error_not_a_wrong_answer():
  cfg = DEFAULT()
  t = weights(cfg, 3)
  engine = make_engine(cfg, t, tokens_per_page=4, num_pages=5, max_len=64)
  engine.step([(0, tokens_for(cfg, 10), [9])])
  with pytest.raises(ValueError):
    engine.step([(1, tokens_for(cfg, 9), [8])])


def test_long_decoding_across_many_pages():
  cfg = DEFAULT()
  toks = tokens_for(cfg, 150)
  t = weights(cfg, 6, toks)
  want = ref.forward(cfg, t, toks)
  engine = make_engine(cfg, t, tokens_per_page=4, num_pages=50)
  assert rel_err(in_portions(engine, toks, [5], slot=3, decode=145), want) < TIGHT


# ---- far keys, edges of windows and blocks, sinks, page borders, the first tokens ------------------------------------------------------

def _peaky(cfg, seed, toks, times=6.0):
  """Scores that spread widely, so that single keys (also far ones, also a pooled block, also the key at a window's edge) carry most
  of a query's weight; slow decays, so that a token hundreds of steps back still matters in the recurrences."""
  t = weights(cfg, seed, toks)
  for i, l in enumerate(cfg["layers"]):
    p = f"l{i}.mix."
    if l["type"] == "attention":
      t[p + "q.norm"] = ref.bf16_values(t[p + "q.norm"] * times)
    else:
      t[p + "A_log"] = ref.bf16_values(t[p + "A_log"] - 5.0)
  return t


@pytest.mark.parametrize("page", [4, 16, 64])
def test_far_keys_and_page_borders(page):
  # blocks of 5 tokens do not divide any of the page sizes; blocks of 4 do
  cfg = model([att(window=0, pool=0, softcap=0.0), dlt(), att(moe(), window=20, pool=5, softcap=40.0), cdl(), att(window=12, pool=4, kv_from=2, softcap=40.0)])
  n = 330
  toks = tokens_for(cfg, n)
  t = _peaky(cfg, 21, toks)
  want = ref.forward(cfg, t, toks)
  engine = make_engine(cfg, t, tokens_per_page=page, num_pages=700 // page + 2, max_len=400)
  assert rel_err(whole(engine, toks), want) < TIGHT
  # a prompt that ends at, one before and one after a page border, then decoding across the next borders
  for cut in (2 * page - 1, 2 * page, 2 * page + 1):
    assert rel_err(in_portions(engine, toks, [cut], decode=page + 3), want[: cut + page + 3]) < TIGHT, cut
  # far keys and far blocks seen from decoded tokens
  got = [engine.step([(2, toks[:310], [])]).cpu().numpy()] + [engine.step([(2, [tok], [0])]).cpu().numpy() for tok in toks[310:]]
  assert rel_err(np.concatenate(got[1:]), want[310:]) < TIGHT


def test_the_far_past_matters_in_these_tests():
  """The check that the test above would see a lost far key, a lost block or a lost state: the oracle fed only the last 100
  tokens differs clearly in every layer kind."""
  for layers in ([att(window=0, pool=0, softcap=0.0)], [att(window=20, pool=5, softcap=40.0)], [dlt()], [cdl()]):
    cfg = model(layers)
    toks = tokens_for(cfg, 330)
    t = _peaky(cfg, 21, toks)
    assert rms_err(ref.forward(cfg, t, toks[230:])[-20:], ref.forward(cfg, t, toks)[-20:]) > 1e-2, layers[0]["type"]


@pytest.mark.parametrize("dtype,tol", [("float32", TIGHT), ("bfloat16", LOOSE)])
@pytest.mark.parametrize("window,pool", [(1, 1), (7, 3), (16, 4), (33, 8), (10, 16)])
def test_keys_just_inside_and_just_outside_the_window_and_blocks_just_seen_and_not_yet(window, pool, dtype, tol):
  """Peaky scores: a query's weight sits on few keys or blocks, often the oldest token it may see or the newest block.  The oracle
  with a window one key wider or narrower, or with one block more or fewer, gives clearly different logits, so an edge that is one
  off would show; the engine agrees with the exact one over a whole prompt, over portions that end around the edges, and decoding
  one token at a time."""
  geo = dict(heads=4, kv_heads=2, dim=16, vdim=16, softcap=50.0)
  cfg = model([att(window=window, pool=pool, **geo), att(moe(), window=window + 2, pool=pool + 1, kv_from=0, **geo)])
  n = 3 * window + 3 * pool + 40
  # every token `pool` times in a row, so that a block's mean key is as telling as a single key
  toks = [tok for tok in tokens_for(cfg, n // pool + 1, seed=window) for _ in range(pool)][:n]
  t = _peaky(cfg, 30 + window, toks, times=10.0)
  want = ref.forward(cfg, t, toks)
  for hook in ({"window": 1}, {"window": -1}, {"blocks": 1}, {"blocks": -1}):
    if window == 1 and hook.get("window") == -1:
      continue
    bad = ref.forward(cfg, t, toks, hooks={0: hook, 1: hook})
    assert rms_err(bad[window + pool :], want[window + pool :]) > 1.5 * LOOSE, hook
  engine = make_engine(cfg, t, dtype=dtype, tokens_per_page=8, num_pages=60)
  err = rel_err if dtype == "float32" else rms_err
  assert err(whole(engine, toks), want) < tol
  for cuts in ([window - 1, 1, 1, window, 2], [window, window + 1, window - 1], [window + pool - 1, 2, 2 * window - 3], [window + pool, pool, 1, pool - 1]):
    cuts = [c for c in cuts if c > 0]
    d = window + 2 * pool + 3
    assert err(in_portions(engine, toks, cuts, decode=d), want[: sum(cuts) + d]) < tol, cuts


@pytest.mark.parametrize("dtype,tol", [("float32", TIGHT), ("bfloat16", LOOSE)])
def test_a_sink_that_outweighs_the_keys(dtype, tol):
  cfg = model([att(heads=4, kv_heads=2, dim=16, vdim=16), att(moe(), heads=8, kv_heads=1, dim=32, vdim=32, window=0, pool=0)])
  toks = tokens_for(cfg, 70)
  t = weights(cfg, 40, toks)
  for i in range(2):
    t[f"l{i}.mix.sink"] = ref.bf16_values(t[f"l{i}.mix.sink"] + 3.0)
  want = ref.forward(cfg, t, toks)
  assert rms_err(ref.forward(cfg, t, toks, hooks={0: {"no_sink": True}, 1: {"no_sink": True}}), want) > 0.05  # leaving the sink out would show
  engine = make_engine(cfg, t, dtype=dtype, tokens_per_page=16, num_pages=20)
  err = rel_err if dtype == "float32" else rms_err
  assert err(whole(engine, toks), want) < tol
  assert err(in_portions(engine, toks, [50], decode=20), want) < tol


def test_first_tokens_of_a_sequence():
  cfg = DEFAULT()
  t = weights(cfg, 9)
  engine = make_engine(cfg, t)
  for n in (1, 2, 3, 4):
    toks = tokens_for(cfg, n, seed=n)
    assert rel_err(whole(engine, toks), ref.forward(cfg, t, toks)) < TIGHT
    # token by token: the rows before the start are zeros, not the rings' old rows
    assert rel_err(in_portions(engine, toks, [], decode=n), ref.forward(cfg, t, toks)) < TIGHT


# ---- other sizes ------------------------------------------------------------------------------------------------------------------

SIZES = {
    "odd_width": lambda: model([att(moe(7, 3, 9, 5)), dlt(moe()), cdl()], width=36, vocab=47, side_dim=3),
    "no_side_input": lambda: model([att(moe()), dlt(moe())], side_dim=0),
    "heads_with_kv_heads_of_their_own": lambda: model([att(kv_heads=4), dlt(kv_heads=4), cdl(kv_heads=4)]),
    "one_head_everywhere": lambda: model([att(heads=1, kv_heads=1), dlt(heads=1, kv_heads=1), cdl(heads=1, kv_heads=1)]),
    "many_heads_on_one_key_head": lambda: model([att(heads=10, kv_heads=1, dim=8, vdim=8), dlt(heads=6, kv_heads=1)]),
    "value_size_over_key_size": lambda: model([att(dim=8, vdim=40), dlt(dim=8, vdim=36), cdl(dim=4, vdim=28)]),
    "key_size_over_value_size": lambda: model([att(dim=40, vdim=4, rot_dims=40), dlt(dim=36, vdim=6), cdl(dim=44, vdim=3)]),
    "rotation_of_two_channels": lambda: model([att(rot_dims=2)]),
    "rotation_of_every_channel": lambda: model([att(rot_dims=12)]),
    "delta_sizes_not_multiples_of_four": lambda: model([dlt(heads=2, kv_heads=1, dim=18, vdim=7), cdl(heads=3, kv_heads=3, dim=9, vdim=11)]),
    "wide_delta_heads": lambda: model([dlt(heads=2, kv_heads=1, dim=136, vdim=24), cdl(heads=1, kv_heads=1, dim=256, vdim=16)], width=64),
    "shared_cache_two_layers_back": lambda: model([att(moe()), dlt(), att(kv_from=0, window=30, pool=2), att(kv_from=0, window=2, pool=3)]),
    "two_taps": lambda: model([dlt(moe(), taps=2), cdl(taps=2)]),
    "seven_taps": lambda: model([dlt(moe(), taps=7), cdl(taps=7)]),
    "more_taps_than_the_convolution_keeps_a_table_for": lambda: model([dlt(taps=20)]),
    "layers_without_feed_forward": lambda: model([att(), dlt(), cdl()]),
    "many_experts_top_one": lambda: model([dlt(moe(40, 1, 6, 0))]),
    "blocks_longer_than_pages": lambda: model([att(window=6, pool=11)]),
    "window_longer_than_the_sequence": lambda: model([att(window=100, pool=4)]),
}


@pytest.mark.parametrize("dtype,tol", [("float32", TIGHT), ("bfloat16", LOOSE)])
@pytest.mark.parametrize("case", sorted(SIZES))
def test_other_sizes(case, dtype, tol):
  # (bfloat16: odd widths and sizes take the unvectorised loads of the tensor-core projections and the row kernel of the attention)
  cfg = SIZES[case]()
  toks = tokens_for(cfg, 41)
  t = weights(cfg, 13, toks)
  want = ref.forward(cfg, t, toks)
  engine = make_engine(cfg, t, dtype=dtype, tokens_per_page=8)
  err = rel_err if dtype == "float32" else rms_err
  assert err(in_portions(engine, toks, [22, 17], slot=0, decode=2), want) < tol


def test_sizes_made_of_whole_tensor_core_tiles_on_a_bfloat16_engine():
  cfg = model([att(moe(8, 2, 128, 128), heads=4, kv_heads=2, dim=64, vdim=64, window=40, pool=8, rot_dims=32),
               dlt(moe(8, 2, 64, 0), heads=4, kv_heads=2, dim=64, vdim=64, taps=4),
               att(moe(4, 2, 128, 64), heads=4, kv_heads=2, dim=64, vdim=64, window=24, pool=8, kv_from=0, rot_dims=32),
               cdl(moe(8, 3, 64, 128), heads=2, kv_heads=2, dim=64, vdim=128, taps=4)], width=128, vocab=256, side_dim=64)
  toks = tokens_for(cfg, 90)
  t = weights(cfg, 15, toks)
  want = ref.forward(cfg, t, toks)
  engine = make_engine(cfg, t, dtype="bfloat16", tokens_per_page=16, num_pages=30)
  assert rms_err(whole(engine, toks), want) < LOOSE
  assert rms_err(in_portions(engine, toks, [70], decode=20), want) < LOOSE


def test_many_rows_per_expert_take_the_pipelined_grouped_products():
  """A prompt portion with at least 128 (row, choice) slots per expert runs its experts on 128-row tiles behind a cp.async ring;
  experts with unequal and odd row counts, a last column tile that is not whole, then single tokens on the small-tile kernel."""
  cfg = model([dlt(moe(3, 2, 72, 0), heads=2, kv_heads=1, dim=32, vdim=32), att(moe(2, 2, 64, 64), heads=2, kv_heads=1, dim=32, vdim=32)], width=128, vocab=200, side_dim=0)
  toks = tokens_for(cfg, 333)
  t = weights(cfg, 25, toks)
  want = ref.forward(cfg, t, toks)
  engine = make_engine(cfg, t, dtype="bfloat16", tokens_per_page=64, num_pages=14, max_len=400)
  assert rms_err(whole(engine, toks), want) < LOOSE
  assert rms_err(in_portions(engine, toks, [301, 2, 27], decode=3), want) < LOOSE


# ---- the tensor-core attention with pooled blocks, cap and sink (bf16, head sizes in multiples of 16) --------------------------------

@pytest.mark.parametrize("heads,kv_heads,dim,page,window,pool", [(4, 2, 64, 16, 70, 8), (2, 2, 16, 8, 33, 3), (8, 1, 32, 64, 20, 1), (6, 2, 48, 4, 64, 5),
                                                                 (4, 1, 128, 32, 40, 16), (12, 1, 96, 16, 9, 2), (2, 1, 256, 16, 50, 7)])
def test_tensor_core_attention_shapes_and_schedules(heads, kv_heads, dim, page, window, pool):
  """Head sizes of the tensor-core arms with a window, pooled blocks (more than one tile of them when the blocks are short), a cap
  and a sink; prompts in portions that end inside, at and after the 64-key tiles, 16-row query tiles that start anywhere, then single
  tokens; peaky scores so that single far blocks matter.  A second layer reads the first one's cache with other edges."""
  geo = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, rot_dims=dim // 2, softcap=50.0)
  cfg = model([att(window=window, pool=pool, **geo), att(moe(), window=window // 2 + 1, pool=pool, kv_from=0, **geo)], width=64, vocab=90, side_dim=8)
  n = 150
  toks = tokens_for(cfg, n, seed=dim)
  t = _peaky(cfg, dim + heads, toks, times=6.0)
  want = ref.forward(cfg, t, toks)
  engine = make_engine(cfg, t, dtype="bfloat16", tokens_per_page=page, num_pages=2 * (n // page + 2) + 2, max_len=n + 8)
  assert rms_err(whole(engine, toks), want) < LOOSE
  for cuts in ([63, 1, 1, 30, 33], [64, 64], [65, 5, 58, 9], [31, 2, 31, 33, 7, 25]):
    assert rms_err(in_portions(engine, toks, cuts, decode=12), want[: sum(cuts) + 12]) < LOOSE, cuts
  # two sequences side by side, one in the middle of its prompt, one decoding
  engine.step([(0, toks[:70], []), (2, toks[:101], [])])
  out = engine.step([(0, toks[70:90], list(range(20))), (2, [toks[101]], [0])]).cpu().numpy()
  assert rms_err(out, np.concatenate([want[70:90], want[101:102]])) < LOOSE


# ---- the framework's entry point: scheduler, sampler -------------------------------------------------------------------------------

def _greedy(cfg, t, prompt, n):
  seq = list(prompt)
  for _ in range(n):
    logits = ref.forward(cfg, t, seq)[-1]
    top2 = np.sort(logits)[-2:]
    assert float(top2[1] - top2[0]) > 1e-4, "near-tie in the test's own model; change the seed"
    seq.append(int(logits.argmax()))
  return seq[len(prompt):]


def test_greedy_generation_through_the_offline_engine():
  from maxtext_indextts2_b200 import offline_engine

  cfg = DEFAULT()
  t = weights(cfg, 17)
  config = pyconfig.from_model_dict(cfg, dtype="float32", per_device_batch_size=2, max_target_length=64, pagedattn_tokens_per_page=4,
                                    pagedattn_num_pages=30, decode_sampling_strategy="greedy")
  eng = offline_engine.OfflineEngine(config, params=as_torch(t))
  prompts = [tokens_for(cfg, n, seed=30 + n) for n in (5, 11, 3, 8, 2)]  # five prompts over two slots: slots, pages and state are reused
  outs = eng.batch_inference(prompts, max_decode_length=9)
  for prompt, out in zip(prompts, outs):
    assert out.token_ids.tolist() == _greedy(cfg, t, prompt, 9)


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
  t = weights(cfg, 19)
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
    assert outs[i] == _greedy(cfg, t, prompt, 6)


@pytest.mark.parametrize("dtype,tol", [("float32", TIGHT), ("bfloat16", 5e-2)])  # (bfloat16: per step, some of few rows)
def test_trace_runner_replays_a_mixed_schedule(tmp_path, dtype, tol):
  import json
  import os
  import subprocess

  cfg = DEFAULT()
  lens = {"a": 70, "b": 9, "c": 33, "d": 5, "e": 40, "f": 20}
  toks = {k: tokens_for(cfg, n, seed=ord(k)) for k, n in lens.items()}
  t = weights(cfg, 23, sum(toks.values(), []))
  model_dir = tmp_path / "model"
  _write_model_dir(model_dir, cfg, t)
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
