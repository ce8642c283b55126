"""Host-side pieces of the Ligidra design: config reading, checks, the plan of layer descriptors.  No GPU."""

import json
import math
import os

import pytest
import torch

from maxtext_indextts2_b200 import ligidra as lg
from maxtext_indextts2_b200 import params as params_lib, pyconfig
from oracle import ligidra_ref as ref
from tests.test_gugidra_host import _write_safetensors

KW = dict(per_device_batch_size=2, max_target_length=40, pagedattn_num_pages=9, pagedattn_tokens_per_page=8)
SCALING = {"factor": 3.0, "low": 1.0, "high": 3.0, "original": 40}


def _model():
  layers = [lg.attention_layer(4, 2, 12, vdim=20, window=9, pool=3, scale=0.31, softcap=6.0, rot_dims=8, rot_base=50.0, rot_scaling=SCALING, mlp=lg.moe_ff(5, 2, 14, 10)),
            lg.delta_layer(4, 2, 12, 10, taps=3, mlp=lg.moe_ff(4, 1, 12)),
            lg.attention_layer(4, 2, 12, vdim=20, window=5, pool=2, scale=0.2, rot_dims=8, rot_base=50.0, kv_from=0),
            lg.delta_layer(2, 1, 8, 6, taps=5, per_channel=True, mlp=lg.moe_ff(6, 3, 10, 8))]
  return lg.model_dict(40, 61, layers, eps=1e-5, side_dim=6)


def test_model_folder_round_trip_and_plan(tmp_path):
  cfg = _model()
  tensors = {k: torch.from_numpy(v).to(torch.bfloat16) for k, v in ref.random_model(cfg, seed=1, rank=5).items()}
  os.makedirs(tmp_path / "m")
  with open(tmp_path / "m" / "config.json", "w") as f:
    json.dump(cfg, f)
  _write_safetensors(tmp_path / "m" / "model.safetensors", tensors)
  loaded = params_lib.load_model_dir(str(tmp_path / "m"))
  assert set(loaded) == set(tensors) and all(torch.equal(loaded[k], v) for k, v in tensors.items())
  config = pyconfig.from_model_dir(str(tmp_path / "m"), **KW)
  assert config.decoder_block == "ligidra" and config.emb_dim == 40 and config.vocab_size == 61 and config.num_decoder_layers == 4
  assert config.token_side_dim == 6 and config.normalization_layer_epsilon == 1e-5
  plan = lg.model_plan(config, loaded)
  assert plan["head"] is plan["embedding"] and torch.equal(plan["embed_norm"], tensors["embed.norm"].float()) and plan["side_embed"].shape == (61, 24)
  p0, p1, p2, p3 = plan["layers"]
  assert all(p["norm_style"] == "pre" and p["conv_taps"] == 2 for p in plan["layers"])
  # the token shift as a two-tap convolution that is added to its input: (shift, -shift)
  assert torch.equal(p0["conv1"][0], tensors["l0.shift"].float()) and torch.equal(p0["conv1"][1], -tensors["l0.shift"].float())
  # attention: q, k, v; norm weights over the whole projections; the means of blocks of three tokens before a window of nine
  a = p0["attn"]
  assert p0["n_in"] == 48 + 24 + 40 and torch.equal(p0["w_in"][48:72], tensors["l0.mix.k"]) and torch.equal(p0["w_in"][72:], tensors["l0.mix.v"])
  assert (a["window"], a["pool"], a["softcap"], a["rot_dims"], a["norm_whole"], a["shared_kv"], a["kv_from"]) == (9, 3, 6.0, 8, 1, 0, None)
  assert a["q_norm"].shape == (48,) and a["k_norm"].shape == (24,) and a["sink"].shape == (4,)
  assert torch.allclose(a["rot_freq"], torch.from_numpy(ref.scaled_frequencies(8, 50.0, SCALING)), rtol=1e-14)
  # a layer that reads another layer's cache projects queries only
  b = p2["attn"]
  assert p2["n_in"] == 48 and (b["shared_kv"], b["kv_from"], b["window"], b["pool"], b["softcap"]) == (1, 0, 5, 2, 0.0) and b["k_norm"] is None and p2["moe"] is None
  assert torch.allclose(b["rot_freq"], torch.tensor([50.0 ** (-2.0 * i / 8) for i in range(4)], dtype=torch.float64), rtol=1e-14)
  # gated delta rule: q, k, v, write strengths, the decay's row per head, the output gate; the convolutions tap-major in fp32
  r = p1["rec"]
  assert r["kind"] == "gdelta" and p1["n_in"] == 24 + 24 + 40 + 4 + 4 + 40 and (r["decay_rank"], r["gate_rank"], r["gate_silu"], r["conv_taps"]) == (0, 0, 1, 3)
  assert torch.equal(p1["w_in"][88:92], tensors["l1.mix.b"]) and torch.equal(p1["w_in"][92:96], tensors["l1.mix.a"]) and torch.equal(p1["w_in"][96:], tensors["l1.mix.g"])
  assert r["conv_w"].shape == (3, 88) and torch.equal(r["conv_w"][:, 24:48], tensors["l1.mix.k.conv"].float().t())
  assert abs(r["q_scale"] - 12**-0.5) < 1e-15 and r["key_eps"] == 1e-6 and r["out_norm"].shape == (40,)
  # per-channel decays and the sigmoid gate come through low ranks that the tensors' shapes give
  c = p3["rec"]
  assert p3["n_in"] == 8 + 8 + 12 + 2 + 5 + 6 and (c["decay_rank"], c["gate_rank"], c["gate_silu"], c["conv_taps"]) == (5, 6, 0, 5)
  assert torch.equal(c["decay_up2"], torch.cat([tensors["l3.mix.a2"]] * 2, dim=1)) and c["w_gate_up"].shape == (12, 6) and c["decay_bias"].shape == (16,)
  # experts: gate and up rows interleaved, stacked; softmax scores used as they are
  m = p0["moe"]
  assert (m["experts"], m["top"], m["ff"], m["shared_ff"], m["score_softmax"], m["plain_weights"], m["act_silu"]) == (5, 2, 14, 10, 1, 1, 1)
  assert m["w_gate_up"].shape == (5, 28, 40) and torch.equal(m["w_gate_up"][3, 0::2], tensors["l0.mlp.e3.gate"]) and torch.equal(m["w_gate_up"][3, 1::2], tensors["l0.mlp.e3.up"])
  assert m["w_down"].shape == (5, 40, 14) and torch.equal(m["shared_down"], tensors["l0.mlp.shared.down"]) and p1["moe"]["shared_ff"] == 0
  # the side input: layer i reads the columns [6 i, 6 i + 6) of the second table
  assert [p["side"]["col"] for p in plan["layers"]] == [0, 6, 12, 18] and torch.equal(p2["side"]["proj"], tensors["l2.side.proj"])


def test_scaled_rot_frequencies():
  f = lg.scaled_rot_frequencies(6, 1000.0, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 8.0})  # wavelengths 6.3, 63, 628; borders at 2 and 8
  s = (8.0 / (2 * math.pi) - 1.0) / 3.0
  assert torch.allclose(f, torch.tensor([(1 - s) / 4.0 + s, 0.1 / 4.0, 0.01 / 4.0], dtype=torch.float64), rtol=1e-13)
  assert lg.scaled_rot_frequencies(2, 10.0, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64.0}).tolist() == [1.0]
  assert torch.allclose(lg.scaled_rot_frequencies(4, 100.0, None), torch.tensor([1.0, 0.1], dtype=torch.float64), rtol=1e-14)


def test_input_projection_is_padded_to_whole_tiles_when_the_width_allows():
  cfg = lg.model_dict(64, 50, [lg.delta_layer(2, 1, 8, 8)])
  config = pyconfig.from_model_dict(cfg, **KW)
  t = lg.random_tensors(config, seed=0)
  plan = lg.model_plan(config, t)["layers"][0]
  n = 8 + 8 + 16 + 2 + 2 + 16
  assert plan["n_in"] == 128 and float(plan["w_in"][n:].float().abs().max()) == 0.0 and plan.get("side") is None
  cfg = lg.model_dict(64, 50, [lg.delta_layer(2, 1, 8, 8)], side_dim=5)
  config = pyconfig.from_model_dict(cfg, **KW)
  side = lg.model_plan(config, lg.random_tensors(config, seed=0))["layers"][0]["side"]
  assert side["gate"].shape == (128, 64) and float(side["gate"][5:].float().abs().max()) == 0.0 and side["proj"].shape == (64, 5)


@pytest.mark.parametrize("break_it,match", [
    (lambda c: c["layers"][0].update(type="conv"), "mixer type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=24), "geometry"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=14), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "window"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][1]["mlp"].update(kind="dense"), "feed-forward kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["token_side"].update(dim=-1), "token_side_dim"),
    (lambda c: c.update(architecture="Other"), "architecture"),
])
def test_bad_configs_are_refused(break_it, match):
  cfg = _model()
  break_it(cfg)
  with pytest.raises(ValueError, match=match):
    pyconfig.from_model_dict(cfg, **KW)


def test_missing_or_misshaped_tensors_are_refused():
  cfg = _model()
  config = pyconfig.from_model_dict(cfg, **KW)
  t = {k: torch.from_numpy(v).to(torch.bfloat16) for k, v in ref.random_model(cfg, seed=1).items()}
  bad = dict(t)
  bad["l0.mix.q.norm"] = bad["l0.mix.q.norm"][:12]  # (a weight per head channel instead of one per channel of the whole projection)
  with pytest.raises(ValueError, match="l0.mix.q.norm"):
    lg.model_plan(config, bad)
  bad = dict(t)
  del bad["l1.shift"]
  with pytest.raises(KeyError):
    lg.model_plan(config, bad)
  bad = dict(t)
  bad["side.embed"] = bad["side.embed"][:, :-1]
  with pytest.raises(ValueError, match="side.embed"):
    lg.model_plan(config, bad)


def test_random_tensors_have_the_names_and_shapes_the_plan_reads():
  cfg = _model()
  cfg["layers"][3]["mixer"]["rank"] = 7
  config = pyconfig.from_model_dict(cfg, **KW)
  t = lg.random_tensors(config, seed=3)
  want = ref.random_model(cfg, seed=0, rank=7)
  assert set(t) == set(want)
  assert all(tuple(t[k].shape) == want[k].shape for k in t if not k.endswith((".g1", ".g2")))  # (the oracle's gate rank is one more than its decay rank)
  lg.model_plan(config, t)
