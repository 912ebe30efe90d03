"""The Viresun configuration, its model description and tensor names, without a GPU."""
import copy

import pytest
import torch

import plain_viresun
from viresun_configs import CONFIGS, VIRESUN_A


def spec_of(config):
    from allpaca_b200.models import resolve
    arch = resolve(config)
    return arch, arch.spec_builder(arch.config_class.from_dict(config))


def test_registered_by_its_name_in_the_singular():
    from allpaca_b200.models import known_architectures
    arch, spec = spec_of(VIRESUN_A)
    assert arch.name == "Viresun" and "Viresun" in known_architectures()
    assert spec.hidden_size == 72 and spec.vocab_size == 211
    # five entries of the order over four layers with tensors: the last runs the second's
    assert len(spec.layers) == 4 and [r.layer for r in spec.order] == [0, 1, 2, 3, 1]
    assert spec.embedding_sinusoid_base == 10000.0 and spec.embedding_norm is not None


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_names_and_shapes(name):
    from allpaca_b200.models import DecoderModel
    from allpaca_b200.parts import BuildEnv, Workspace
    config = CONFIGS[name]
    _, spec = spec_of(config)
    cpu = torch.device("cpu")
    model = DecoderModel(spec, BuildEnv(torch.float32, cpu, Workspace(cpu)))
    targets = {k: tuple(v[0].shape) for k, v in model.weight_targets().items()}
    assert targets == plain_viresun.tensor_shapes(config)


def test_caches_and_states_per_run_of_the_order():
    from allpaca_b200.models import DecoderModel
    from allpaca_b200.parts import BuildEnv, Workspace
    _, spec = spec_of(VIRESUN_A)
    cpu = torch.device("cpu")
    model = DecoderModel(spec, BuildEnv(torch.float32, cpu, Workspace(cpu), page_size=8))
    plan = model.cache_plan()
    # the two attention layers of equal shape share a pool, the one with another window has its own
    assert [g.runs for g in plan] == [[0, 2], [3]]
    assert plan[0].need.window == 21 and plan[0].need.page_shape(8) == (2, 8, 24 + 40)
    assert plan[1].need.window == 5 and plan[1].need.page_shape(8) == (4, 8, 32)
    # both runs of the Mamba layer keep a state of their own: 6 heads x 20 x 12 and 3 inputs of 192 channels
    per_run = 4 * (6 * 20 * 12 + 3 * (72 + 2 * 3 * 20))
    assert model.state_bytes() == [0, per_run, 0, 0, per_run]
    assert not model.host_control()


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="lstm"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "multiple"),
    (lambda c: c["layers"][1]["mixer"].update(groups=4), "multiple"),
    (lambda c: c["layers"][1]["mixer"].update(norm_groups=5), "equal parts"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "chosen"),
    (lambda c: c["layers"][4].update(weights_of=4), "earlier"),
    (lambda c: c["layers"][4]["mixer"].update(state=21), "another layer"),
    (lambda c: c.update(width=71), "even"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
])
def test_configurations_that_are_refused(change, message):
    from allpaca_b200.config import ConfigError, ViresunConfig
    config = copy.deepcopy(VIRESUN_A)
    change(config)
    with pytest.raises(ConfigError, match=message):
        ViresunConfig.from_dict(config)


def test_plain_prefix_property():
    """The plain implementation is causal: a prefix's logits do not change when tokens follow."""
    config = CONFIGS["A"]
    w = plain_viresun.random_tensors(config, 1)
    tokens = torch.randint(0, config["vocab"], (40,), generator=torch.Generator().manual_seed(0)).tolist()
    whole = plain_viresun.forward(config, w, tokens)
    part = plain_viresun.forward(config, w, tokens[:27])
    assert float((whole[:27] - part).abs().max()) < 1e-9


def test_random_model_folder_from_the_command_line(tmp_path):
    """``allpaca init-random --config`` writes a Viresun folder the engine's reader accepts: every tensor
    the description names, the numbers inside the bias's logarithm positive, the norms' weights one
    number each."""
    import json
    from allpaca_b200 import cli
    from allpaca_b200.models import load_config
    from allpaca_b200.weights.safetensors_io import Checkpoint
    src = tmp_path / "config.json"
    src.write_text(json.dumps(VIRESUN_A))
    assert cli.main(["init-random", "--config", str(src), "--seed", "3", "--out", str(tmp_path / "m"),
                     "--dtype", "bfloat16"]) == 0
    arch, cfg = load_config(str(tmp_path / "m"))
    assert arch.name == "Viresun" and cfg.torch_dtype == "bfloat16" and len(cfg.layers) == 5
    ckpt = Checkpoint(str(tmp_path / "m"))
    assert set(ckpt.names()) == set(plain_viresun.tensor_shapes(VIRESUN_A))
    assert float(ckpt.tensor("l0.mix.r2").float().min()) > 0 and float(ckpt.tensor("l3.mix.r1").float().min()) > 0
    assert tuple(ckpt.tensor("l1.norm2").shape) == ()
