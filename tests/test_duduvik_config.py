"""
Host-side tests of the Duduvik architecture: config.json parsing, the model description it turns
into, tensor names, sizes read from the checkpoint, what the cache is asked for, and two checks of
the plain implementation against closed forms.
"""

import copy

import pytest
import torch

import duduvik_configs as C
import plain_duduvik as plain


def spec_of(raw):
    from tinyserve_llm_b200.config import resolve_architecture
    arch = resolve_architecture(raw)
    return arch.spec(arch.parse(raw))


def test_the_architecture_is_found_by_its_name_and_layers_keep_their_order():
    spec = spec_of(C.MIXED)
    assert spec.architecture == "Duduvik" and spec.vocab_size == 300 and spec.hidden_size == 96
    assert spec.embedding_scale == 7.0 and spec.lm_head_name is None and spec.embedding_name == "embed"
    kinds = [(b.mixer.kind, None if b.feed_forward is None else b.feed_forward.kind) for b in spec.blocks]
    assert kinds == [("linear_recurrence", "routed_experts"), ("latent_attention", "gated_mlp"),
                     ("linear_recurrence", None), ("latent_attention", "routed_experts"), ("linear_recurrence", "gated_mlp")]
    assert all(b.arrangement == "sandwich_norm" for b in spec.blocks)
    gla, att, ret = spec.blocks[0].mixer, spec.blocks[1].mixer, spec.blocks[2].mixer
    assert (gla.decay, gla.tau, gla.q_scale, gla.k_scale) == ("channel_logits", 8.0, 24 ** -0.5, 1.0)
    assert (ret.decay, ret.head_decays, ret.k_scale, ret.position.dims, ret.position.base) == (
        "head", (0.9, 0.97, 0.995), 32 ** -0.5, 16, 5000.0)
    assert (att.window, att.scale, att.kv_rank, att.rot_dim, att.norm_eps) == (21, 0.2, 48, 8, 1e-5)
    moe = spec.blocks[0].feed_forward
    assert (moe.num_experts, moe.top, moe.expert.limit, moe.expert.alpha, moe.shared.intermediate_size) == (6, 3, 2.0, 1.702, 56)
    assert spec.blocks[3].feed_forward.shared is None and spec.blocks[4].feed_forward.activation == "relu"


def test_declared_tensors_carry_the_checkpoint_names():
    from tinyserve_llm_b200.parts.model import declared_tensors
    d = declared_tensors(spec_of(C.MIXED))
    for name, shape in {"embed": (300, 96), "final.norm": (96,), "l0.norm1": (96,), "l0.norm2b": (96,),
                        "l0.mix.a1": (12, 96), "l0.mix.a2": (48, 12), "l0.mix.a2.b": (48,), "l0.mix.norm": (40,),
                        "l0.mlp.e5.gate": (40, 96), "l0.mlp.router.b": (6,), "l0.mlp.shared.down": (96, 56),
                        "l1.mix.dkv": (56, 96), "l1.mix.dkv.norm": (48,), "l1.mix.uq": (72, 40), "l1.mix.uk": (48, 48),
                        "l1.mix.uv": (72, 48), "l1.mlp.down": (96, 136), "l2.mix.g": (48, 96)}.items():
        assert tuple(d[name].shape) == shape, name
    assert "l2.norm2" not in d and "l2.mlp.gate" not in d and "l2.mix.norm" not in d      # no feed-forward; a norm without weight
    assert "l3.mlp.shared.gate" not in d


def test_a_size_the_configuration_does_not_give_is_read_from_the_checkpoint(tmp_path):
    """The inner size of the low-rank decay projection: any value loads, a mismatch between its two tensors does not."""
    from tinyserve_llm_b200.parts.model import declared_tensors
    from tinyserve_llm_b200.weights import load_tensors, write_random_model
    from tinyserve_llm_b200.weights.loader import CheckpointError
    raw = copy.deepcopy(C.RECURRENT)
    write_random_model(str(tmp_path), raw, 1)
    del raw["layers"][1]["mixer"]["decay_rank"]
    declared = declared_tensors(spec_of(raw))
    assert tuple(declared["l1.mix.a1"].shape) == (-1, 64)
    tensors = load_tensors(str(tmp_path), declared)
    assert tuple(tensors["l1.mix.a1"].shape) == (8, 64) and tuple(tensors["l1.mix.a2"].shape) == (40, 8)
    with pytest.raises(ValueError, match="takes a size from the checkpoint"):
        write_random_model(str(tmp_path / "x"), raw, 1)
    wrong = copy.deepcopy(C.RECURRENT)
    wrong["layers"][1]["mixer"]["heads"] = 2
    with pytest.raises(CheckpointError):
        load_tensors(str(tmp_path), declared_tensors(spec_of(wrong)))


@pytest.mark.parametrize("edit, needle", [
    (lambda r: r["layers"][0].update(type="conv"), "not supported"),
    (lambda r: r["layers"][2]["mixer"].update(decay=[0.5]), "entries for 3 heads"),
    (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=6), "differs from rot_dim"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=7), "exceeds experts"),
    (lambda r: r.pop("width"), "lacks 'width'"),
    (lambda r: r["layers"][4]["mlp"].update(kind="conv"), "not supported"),
    (lambda r: r["layers"][2]["mixer"]["rot"].update(dims=34), "exceeds dim"),
])
def test_bad_configurations_are_refused_with_the_reason(edit, needle):
    from tinyserve_llm_b200.config import ConfigError
    raw = copy.deepcopy(C.MIXED)
    edit(raw)
    with pytest.raises(ConfigError, match=needle):
        spec_of(raw)


def test_the_cache_is_asked_for_latent_rows_and_state_slots():
    """Attention layers: one row of kv_rank + rot_dim per token, no value pool, a group per window; recurrences: a slot."""
    from tinyserve_llm_b200.cache.manager import CacheManager, plan_layout
    from tinyserve_llm_b200.parts.base import KVNeed
    needs = [(None, 2 * 24 * 40 * 4), (KVNeed(1, 56, 21, values=False), 0), (None, 3 * 32 * 16 * 4),
             (KVNeed(1, 48, 50, values=False), 0), (None, 3 * 16 * 16 * 4)]
    layout = plan_layout(needs, 16)
    assert [(g.entries, g.head_dim, g.window, g.values) for g in layout.groups] == [((1,), 56, 21, False), ((3,), 48, 50, False)]
    assert layout.state_offsets[1] == -1 and layout.state_offsets[0] == 0 and layout.state_bytes >= sum(n[1] for n in needs)
    manager = CacheManager(layout, 8, num_state_slots=2)
    assert len(manager.pools) == 2 and not manager.caching
    assert manager.admit("a", list(range(40))) and manager.admit("b", [1, 2, 3])
    assert not manager.admit("c", [1])                                              # both slots are taken
    manager.commit("a", 40)
    assert manager.block_table("a", 0) == [-1, manager.block_table("a", 0)[1], manager.block_table("a", 0)[2]]   # window 21: page 0 passed
    assert -1 not in manager.block_table("a", 1)                                    # window 50: nothing passed yet
    recurrent = plan_layout([(None, 100), (None, 300)], 16)
    manager = CacheManager(recurrent, 8, num_state_slots=1)                         # no pages at all
    assert manager.pools == [] and manager.admit("x", list(range(1000))) and manager.available_pages() == ()


def test_plain_retention_equals_its_closed_form():
    """o_t = sum_(j<=t) decay^(t-j) (q_t . k_j) v_j, then the norm, gate and projection."""
    g = torch.Generator().manual_seed(0)
    m = {"heads": 2, "dim": 6, "vdim": 5, "decay": [0.8, 0.95], "rot": {"dims": 4, "base": 30.0}}
    w = {k: torch.randn(s, generator=g, dtype=torch.float64) for k, s in
         {"q": (12, 9), "k": (12, 9), "v": (10, 9), "g": (10, 9), "o": (9, 10)}.items()}
    h = torch.randn(11, 9, generator=g, dtype=torch.float64)
    pos = torch.arange(11)
    got = plain.mixer_retention(m, w, h, pos, 1e-6)
    q = plain.rotate_half((h @ w["q"].T).view(11, 2, 6), pos, 4, 30.0)
    k = plain.rotate_half((h @ w["k"].T).view(11, 2, 6), pos, 4, 30.0) * 6 ** -0.5
    v = (h @ w["v"].T).view(11, 2, 5)
    o = torch.zeros(11, 2, 5, dtype=torch.float64)
    for t in range(11):
        for j in range(t + 1):
            for hd in range(2):
                o[t, hd] += m["decay"][hd] ** (t - j) * (q[t, hd] @ k[j, hd]) * v[j, hd]
    o = plain.rms_unit(o, 1e-6).reshape(11, 10)
    gate = h @ w["g"].T
    torch.testing.assert_close(got, (o * gate * torch.sigmoid(gate)) @ w["o"].T)


def test_plain_rotation_turns_pairs_and_leaves_the_rest():
    x = torch.arange(12, dtype=torch.float64).view(1, 1, 12) + 1
    y = plain.rotate_half(x, torch.tensor([3]), 4, 100.0)
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    want = [1 * torch.cos(torch.tensor(a0)) - 3 * torch.sin(torch.tensor(a0)), 2 * torch.cos(torch.tensor(a1)) - 4 * torch.sin(torch.tensor(a1)),
            3 * torch.cos(torch.tensor(a0)) + 1 * torch.sin(torch.tensor(a0)), 4 * torch.cos(torch.tensor(a1)) + 2 * torch.sin(torch.tensor(a1))]
    torch.testing.assert_close(y[0, 0, :4], torch.stack(want).double())
    assert torch.equal(y[0, 0, 4:], x[0, 0, 4:])
