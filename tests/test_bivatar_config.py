"""The Bivatar configuration and model description without a GPU: tensor names and shapes against the
plain list, the cache plan, stretched rotary frequencies against the plain formula, refused
configurations, and windowed page groups that keep a request's first pages."""
import copy
import math

import pytest
import torch

import plain_bivatar
from bivatar_configs import CONFIGS, ONLY_LATENT

from allpaca_b200.cache import CacheManager, GroupLayout
from allpaca_b200.config import ConfigError
from allpaca_b200.models import DecoderModel, resolve
from allpaca_b200.parts import BuildEnv, Workspace
from allpaca_b200.parts.rope import inverse_frequencies, magnitude


def build(config, dtype=torch.float32):
    arch = resolve(config)
    cfg = arch.config_class.from_dict(config)
    env = BuildEnv(dtype=dtype, device=torch.device("cpu"), workspace=Workspace(torch.device("cpu")), page_size=8)
    return cfg, DecoderModel(arch.spec_builder(cfg), env)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_names_and_shapes(name):
    _, model = build(CONFIGS[name])
    got = {n: tuple(ws.shape) for n, (ws, _, _) in model.weight_targets().items()}
    assert got == plain_bivatar.tensor_shapes(CONFIGS[name])


def test_cache_plan_shares_latents_and_keeps_first_tokens():
    _, model = build(CONFIGS["A"])
    plan = model.cache_plan()
    needs = [(g.need.outer, g.need.inner, g.need.window, g.need.keep_first, g.runs) for g in plan]
    assert needs == [((), (64,), None, 0, [0]), ((2,), (64,), 21, 5, [1]), ((), (48,), None, 0, [3]),
                     ((4,), (32,), 5, 0, [4])]
    order = model.spec.order
    assert [(r.layer, r.cache_from) for r in order] == [(0, None), (1, None), (2, 0), (3, None), (4, None), (5, 3)]
    assert model.state_bytes() == [0] * 6 and not model.host_control()


@pytest.mark.parametrize("dims,base,scaling", [(16, 10000.0, (4.0, 64, 8.0, 1.0)), (8, 1000.0, (16.0, 32, 4.0, 0.5)),
                                               (6, 50.0, (2.0, 16, 2.0, 0.25)), (64, 50000.0, (40.0, 4096, 32.0, 1.0)),
                                               (8, 500.0, None)])
def test_stretched_frequencies(dims, base, scaling):
    named = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
    want, grow = plain_bivatar.stretched_frequencies(dims, base, named)
    part = dict(named, rope_type="yarn") if named else None
    got = inverse_frequencies(dims, base, part)
    assert torch.allclose(got, torch.tensor(want, dtype=torch.float64), rtol=1e-12, atol=0)
    assert math.isclose(magnitude(part), grow, rel_tol=1e-12)


def test_refused_configurations():
    arch = resolve(CONFIGS["A"])

    def broken(change):
        c = copy.deepcopy(CONFIGS["A"])
        change(c)
        with pytest.raises(ConfigError):
            arch.config_class.from_dict(c)
    broken(lambda c: c["layers"][2]["mixer"].update(kv_from=1))          # not a latent layer
    broken(lambda c: c["layers"][2]["mixer"].update(kv_from=2))          # itself
    broken(lambda c: c["layers"][5]["mixer"].update(kv_from=2))          # a layer that has no latent of its own
    broken(lambda c: c["layers"][2]["mixer"].update(kv_rank=40))         # another latent width than its source
    broken(lambda c: c["layers"][2]["mixer"].update(rot={"dims": 16, "base": 7.0}))    # another rotation than its source
    broken(lambda c: c["layers"][1]["mixer"].update(kv_heads=4))         # 6 heads on 4
    broken(lambda c: c["layers"][3]["mixer"]["rot"].update(dims=7))
    broken(lambda c: c["layers"][3]["mixer"]["rot"].update(dims=10))     # more than rot_dim
    broken(lambda c: c["layers"][0].update(type="mamba2"))
    broken(lambda c: c["norm"].update(eps=0))
    broken(lambda c: c["layers"][0]["mlp"].update(kind="moe"))
    broken(lambda c: c.update(layers=[]))


def test_what_a_configuration_may_leave_out():
    c = copy.deepcopy(ONLY_LATENT)
    del c["residual_mult"], c["embedding"]
    cfg, model = build(c)
    assert cfg.residual_mult == 1.0 and cfg.embedding_scale == 1.0
    assert cfg.layers[0].mixer.rot.scaling is None


def test_window_release_keeps_the_first_pages():
    m = CacheManager([GroupLayout(4, 40), GroupLayout(4, 40, window=6, keep_first=5), GroupLayout(4, 40, window=6)], max_seqs=1)
    m.begin("r")
    m.append("r", 30)
    freed = m.release_passed("r")
    t0, t1, t2 = (m.block_table("r", g) for g in range(3))
    # the next row sits at 30 and sees keys from 25 on: pages 0..5 are passed; the first two hold kept tokens
    assert all(p >= 0 for p in t0)
    assert [p >= 0 for p in t1] == [True, True, False, False, False, False, True, True]
    assert [p >= 0 for p in t2] == [False] * 6 + [True, True]
    assert freed == 4 + 6
    m.check()
    m.free("r")
    m.check()
    assert m.num_free_pages(1) == 40


def test_random_model_folder_from_the_command_line(tmp_path):
    """``allpaca init-random --config`` writes a Bivatar folder the engine's reader accepts: every tensor the
    description names and no other (a layer that reads another's latent has no down-projection to it)."""
    import json
    from allpaca_b200 import cli
    from allpaca_b200.models import load_config
    from allpaca_b200.weights.safetensors_io import Checkpoint
    src = tmp_path / "config.json"
    src.write_text(json.dumps(CONFIGS["A"]))
    assert cli.main(["init-random", "--config", str(src), "--seed", "3", "--out", str(tmp_path / "m"),
                     "--dtype", "bfloat16"]) == 0
    arch, cfg = load_config(str(tmp_path / "m"))
    assert arch.name == "Bivatar" and cfg.torch_dtype == "bfloat16" and len(cfg.layers) == 6
    ckpt = Checkpoint(str(tmp_path / "m"))
    shapes = plain_bivatar.tensor_shapes(CONFIGS["A"])
    assert set(ckpt.names()) == set(shapes)
    assert "l2.mix.dkv" not in shapes and tuple(ckpt.tensor("l3.mix.dkv").shape) == (48, 64)
