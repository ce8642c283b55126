"""Host-side pieces of the Ginodra design: config reading, checks, the plan of layer descriptors.  No GPU."""

import json
import os

import pytest
import torch

from maxtext_indextts2_b200 import ginodra as gi
from maxtext_indextts2_b200 import params as params_lib, pyconfig
from oracle import ginodra_ref as ref
from tests.test_gugidra_host import _write_safetensors

KW = dict(per_device_batch_size=2, max_target_length=40, pagedattn_num_pages=9, pagedattn_tokens_per_page=8)


def _model():
  layers = [gi.delta_layer(3, 12, mlp=gi.dense_ff(56)), gi.attention_layer(4, 2, 24, vdim=20, window=9, scale=0.31, mlp=gi.dense_ff(32)),
            gi.attention_layer(4, 2, 24, vdim=20, window=5, scale=0.2, kv_from=1), gi.latent_layer(3, 12, 8, 20, 10, 28, rot_base=100.0, scale=0.27, mlp=gi.dense_ff(48))]
  return gi.model_dict(40, 61, layers, eps=1e-5, groups=2, taps=3, residual_mult=0.4, logit_scale=0.7, logit_softcap=4.0)


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
  assert config.decoder_block == "ginodra" and config.emb_dim == 40 and config.vocab_size == 61 and config.num_decoder_layers == 4
  assert (config.norm_groups, config.input_conv_taps, config.residual_multiplier, config.logits_scale, config.final_logits_soft_cap) == (2, 3, 0.4, 0.7, 4.0)
  plan = gi.model_plan(config, loaded)
  assert plan["head"] is plan["embedding"] and plan["norm_groups"] == 2 and plan["logit_scale"] == 0.7
  p0, p1, p2, p3 = plan["layers"]
  assert all(p["norm_style"] == "parallel" and p["conv_taps"] == 3 and p["residual_mult"] == 0.4 for p in plan["layers"])
  # delta rule: r, k, v, output gate, removal, then the decay's down-projection; the up-projection transposed, in fp32
  assert p0["rec"]["kind"] == "delta" and p0["n_in"] == 5 * 36 + 5 and p0["rec"]["decay_rank"] == 5
  assert torch.equal(p0["w_in"][36:72], tensors["l0.mix.k"]) and torch.equal(p0["w_in"][144:180], tensors["l0.mix.a"]) and torch.equal(p0["w_in"][180:], tensors["l0.mix.w1"])
  assert torch.equal(p0["rec"]["decay_up_t"], tensors["l0.mix.w2"].float().t()) and torch.equal(p0["rec"]["gate_bias"], tensors["l0.mix.a.b"].float())
  assert abs(p0["rec"]["decay_rate"] - 0.6065306597126334) < 1e-15 and p0["rec"]["key_eps"] == 1e-6
  # the mixer's output projection and the feed-forward's down-projection share one matrix along their inputs
  assert p0["wo"].shape == (40, 36 + 56) and torch.equal(p0["wo"][:, :36], tensors["l0.mix.o"]) and torch.equal(p0["wo"][:, 36:], tensors["l0.mlp.down"])
  assert torch.equal(p0["conv1"], tensors["l0.canon1"].float().t()) and torch.equal(p0["conv2"][2], tensors["l0.canon2"].float()[:, 2])
  # attention: q, k, v, head gates; slopes 2^(-8 (h + 1) / H)
  a = p1["attn"]
  assert p1["n_in"] == 96 + 48 + 40 + 4 and torch.equal(p1["w_in"][144:184], tensors["l1.mix.v"]) and torch.equal(p1["w_in"][184:], tensors["l1.mix.g"])
  assert (a["window"], a["shared_kv"], a["head_gate"], a["rot_dims"], a["kv_from"]) == (9, 0, 1, 0, None)
  assert a["slopes"].tolist() == [0.25, 0.0625, 0.015625, 0.00390625] and a["sink"] is None
  # a layer that reads another layer's cache projects queries and gates only
  b = p2["attn"]
  assert p2["n_in"] == 96 + 4 and (b["shared_kv"], b["kv_from"], b["window"]) == (1, 1, 5) and b["k_norm"] is None and p2["ff"] == 0 and p2["conv2"] is None
  assert p2["wo"].shape == (40, 80)
  # latent attention: the key expansion is stored per head, transposed
  l = p3["latent"]
  assert p3["n_in"] == 10 + 36 + 3 and torch.equal(p3["w_in"][10:46], tensors["l3.mix.dkv"]) and l["rot_half"] == 1
  assert l["w_uk_t"].shape == (3, 28, 12) and torch.equal(l["w_uk_t"][1], tensors["l3.mix.uk"][12:24].t()) and l["w_uv"].shape == (3, 20, 28)
  assert torch.allclose(l["rot_freq"], torch.tensor([100.0 ** (-2.0 * i / 8) for i in range(4)], dtype=torch.float64), rtol=1e-14)


def test_input_projection_is_padded_to_whole_tiles_when_the_width_allows():
  cfg = gi.model_dict(64, 50, [gi.delta_layer(2, 8)])
  config = pyconfig.from_model_dict(cfg, **KW)
  t = gi.random_tensors(config, seed=0)
  plan = gi.model_plan(config, t)["layers"][0]
  n = 5 * 16 + 16
  assert plan["n_in"] == 128 and float(plan["w_in"][n:].float().abs().max()) == 0.0


@pytest.mark.parametrize("break_it,match", [
    (lambda c: c["layers"][0].update(type="conv"), "mixer type"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=0), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=24), "geometry"),
    (lambda c: c["layers"][3]["mixer"]["rot"].update(dims=4), "rot_dim"),
    (lambda c: c["layers"][3]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mlp"].update(kind="moe"), "feed-forward kind"),
    (lambda c: c["norm"].update(groups=3), "norm_groups"),
    (lambda c: c["canon"].update(taps=-1), "input_conv_taps"),
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
  bad["l3.mix.dkv.norm"] = bad["l3.mix.dkv.norm"][:-1]
  with pytest.raises(ValueError, match="l3.mix.dkv.norm"):
    gi.model_plan(config, bad)
  bad = dict(t)
  del bad["l1.canon2"]
  with pytest.raises(KeyError):
    gi.model_plan(config, bad)


def test_random_tensors_have_the_names_and_shapes_the_plan_reads():
  cfg = _model()
  config = pyconfig.from_model_dict(cfg, **KW)
  t = gi.random_tensors(config, seed=3)
  want = ref.random_model(cfg, seed=0, rank=16)
  assert set(t) == set(want) and all(tuple(t[k].shape) == want[k].shape for k in t)
  gi.model_plan(config, t)
