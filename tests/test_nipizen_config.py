"""Host-side tests of the Nipizen configuration, its model description and the plain implementation."""

import copy

import pytest
import torch

import nipizen_configs as C
import plain_nipizen as plain
from tinyserve_llm_b200.config import ConfigError
from tinyserve_llm_b200.config.nipizen import NipizenConfig, nipizen_model_spec
from tinyserve_llm_b200.config.registry import resolve_architecture
from tinyserve_llm_b200.config.spec import GatedAttentionSpec, GatedDeltaRuleSpec, MatrixLSTMSpec, ParallelMixerSpec
from tinyserve_llm_b200.parts.model import declared_tensors
from tinyserve_llm_b200.parts.rotary import yarn_frequencies
from tinyserve_llm_b200.weights import random_tensors


def test_every_size_and_constant_comes_from_the_configuration():
    config = NipizenConfig.from_dict(C.MIXED)
    spec = nipizen_model_spec(config)
    assert resolve_architecture(C.MIXED).name == "Nipizen"
    assert spec.vocab_size == 300 and spec.hidden_size == 96 and len(spec.blocks) == 4 and spec.lm_head_name is None
    first = spec.blocks[0].mixer
    assert isinstance(first, ParallelMixerSpec) and [b[1] for b in first.branches] == ["left.", "right."]
    left, right = first.branches[0][0], first.branches[1][0]
    assert isinstance(left, GatedAttentionSpec) and isinstance(right, GatedDeltaRuleSpec)
    assert (left.num_heads, left.num_kv_heads, left.head_dim, left.value_dim, left.scale) == (4, 2, 24, 40, 0.2)
    assert left.position.dims == 16 and left.position.base == 5000.0 and left.position.yarn.factor == 4.0
    assert left.bias and left.qk_norm and left.output_gate and left.qk_norm_eps == 1e-5
    assert (right.num_heads, right.num_kv_heads, right.key_dim, right.value_dim, right.conv_taps) == (4, 2, 20, 24, 3)
    assert right.q_scale == 20 ** -0.5 and (first.branches[0][2], first.branches[1][2]) == (0.7, 1.3)
    second = spec.blocks[1].mixer
    assert isinstance(second, MatrixLSTMSpec) and second.gate_cap == 10.0 and second.q_scale == 24 ** -0.5
    assert spec.blocks[2].feed_forward is None and spec.blocks[2].mixer.branches[0][0].position.yarn is None
    experts = spec.blocks[0].feed_forward
    assert (experts.num_experts, experts.top, experts.scoring, experts.weight_on) == (6, 2, "sigmoid", "input")
    assert experts.expert.intermediate_size == 40 and experts.expert.activation == "relu2"


def test_declared_tensors_follow_the_sizes():
    d = declared_tensors(nipizen_model_spec(NipizenConfig.from_dict(C.MIXED)))
    assert d["embed"].shape == (300, 96) and d["final.norm"].shape == (96,) and d["l0.norm2"].shape == (96,)
    assert d["l0.mix.left.q"].shape == (96, 96) and d["l0.mix.left.k.b"].shape == (48,) and d["l0.mix.left.v"].shape == (80, 96)
    assert d["l0.mix.left.q.norm"].shape == (96,) and d["l0.mix.left.g"].shape == (160, 96) and d["l0.mix.left.o"].shape == (96, 160)
    assert d["l0.mix.right.q.conv"].shape == (40, 3) and d["l0.mix.right.v.conv"].shape == (96, 3)
    assert d["l0.mix.right.a2"].shape == (80, 10) and d["l0.mix.right.dt_bias"].shape == (80,) and d["l0.mix.right.g2"].shape == (96, 6)
    assert d["l0.mix.right.b"].shape == (4, 96) and d["l0.mix.right.norm"].shape == (24,) and d["l0.mix.right.A_log"].shape == (4,)
    assert d["l1.mix.norm"].shape == (120,) and d["l1.mix.i.b"].shape == (3,) and d["l1.mix.o"].shape == (96, 120)
    assert d["l1.mlp.e4.up"].shape == (24, 96) and d["l1.mlp.router"].shape == (5, 96) and "l1.mlp.router.b" not in d
    assert not any(n.startswith("l2.mlp.") or n == "l2.norm2" for n in d)
    raw = copy.deepcopy(C.MIXED)
    del raw["layers"][0]["mixer"]["right"]["decay_rank"]                     # the size is then the checkpoint's
    assert declared_tensors(nipizen_model_spec(NipizenConfig.from_dict(raw)))["l0.mix.right.a1"].shape == (-1, 96)


@pytest.mark.parametrize("edit, message", [
    (lambda r: r["layers"][0].update(type="attention"), "layers[0].type"),
    (lambda r: r["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
    (lambda r: r["layers"][0]["mixer"]["left"]["rot"].update(dims=26), "rot.dims"),
    (lambda r: r["layers"][1]["mixer"].pop("gate_cap"), "gate_cap"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=9), "top"),
    (lambda r: r["layers"][0]["mixer"].pop("right_scale"), "right_scale"),
    (lambda r: r.pop("width"), "width"),
])
def test_what_cannot_be_served_is_refused_with_the_key(edit, message):
    raw = copy.deepcopy(C.MIXED)
    edit(raw)
    with pytest.raises(ConfigError, match=message.replace("[", r"\[").replace("]", r"\]")):
        NipizenConfig.from_dict(raw)


def test_yarn_frequencies_against_the_plain_ones():
    from tinyserve_llm_b200.config.spec import YarnScaling
    for dims, base, scaling in ((16, 5000.0, (4.0, 64, 16.0, 2.0)), (32, 10000.0, (8.0, 128, 32.0, 1.0)), (8, 100.0, None)):
        rot = {"dims": dims, "base": base}
        if scaling:
            rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
        want, magnitude = plain.rotary_frequencies(rot)
        got = yarn_frequencies(dims, base, YarnScaling(*scaling) if scaling else None)
        torch.testing.assert_close(got, want, atol=0, rtol=1e-12)
        assert magnitude == (1.0 if not scaling else 0.1 * torch.log(torch.tensor(scaling[0], dtype=torch.float64)).item() + 1.0)
    # the ramp is not flat: some frequencies are kept, some divided by the factor, some in between
    f, _ = plain.rotary_frequencies({"dims": 32, "base": 10000.0, "scaling": {"factor": 8.0, "original": 128, "fast": 32.0, "slow": 1.0}})
    ratio = f / (10000.0 ** (-2.0 * torch.arange(16, dtype=torch.float64) / 32))
    assert float(ratio.max()) == 1.0 and abs(float(ratio.min()) - 0.125) < 1e-12 and ((ratio > 0.13) & (ratio < 0.99)).any()


def test_the_plain_model_does_not_depend_on_later_tokens_and_reads_far_ones():
    """Causality of every mechanism of the plain implementation, and a state that carries the first token to the last."""
    raw = C.MIXED
    tensors = dict(random_tensors(declared_tensors(nipizen_model_spec(NipizenConfig.from_dict(raw))), 5, **C.WEIGHTS))
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, raw["vocab"], (40,), generator=g).tolist()
    full = plain.forward(raw, tensors, ids)
    torch.testing.assert_close(plain.forward(raw, tensors, ids[:17]), full[:17], atol=1e-10, rtol=1e-10)
    other = list(ids)
    other[0] = (ids[0] + 1) % raw["vocab"]
    assert float((plain.forward(raw, tensors, other)[-1] - full[-1]).abs().max()) > 1e-6
