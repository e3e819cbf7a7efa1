"""
The Duduvik decoder in the engine against the plain implementation of tests/plain_duduvik.py:
whole prompts, prompts against token-by-token decoding, portions down to two tokens, unequal
requests in one batch against each alone, pages and state slots that are freed and taken again,
windows' edges, far keys, the first tokens, long decoding, several sizes, steps replayed from CUDA
graphs, the replay program and greedy generation through the engine's entry point.
"""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import duduvik_configs as C
import plain_duduvik as plain

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CONFIGS = {"mixed": C.MIXED, "recurrent": C.RECURRENT, "latent_only": C.LATENT_ONLY, "wide": C.WIDE}
SEEDS = {"mixed": 101, "recurrent": 202, "latent_only": 303, "wide": 404}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from tinyserve_llm_b200.weights import write_random_model
    from tinyserve_llm_b200.weights.safetensors_io import write_safetensors
    out = {}
    for name, raw in CONFIGS.items():
        folder = str(tmp_path_factory.mktemp(f"duduvik_{name}"))
        write_random_model(folder, raw, SEEDS[name], **C.WEIGHTS)
        out[name, "float32"] = folder
        # For the bfloat16 comparisons the router's weights are made small beside its bias: the choice of
        # experts then hardly rests on bfloat16's rounding of a token's activations.  With the weights as
        # drawn, a token in a hundred has two router logits closer than that rounding, takes another expert
        # than the float64 model and is compared with the wrong thing (routing of every kind is compared
        # exactly in float32, and in bfloat16 by the test of the routed feed-forward alone).
        steady = str(tmp_path_factory.mktemp(f"duduvik_{name}_steady"))
        tensors = read_tensors(folder)
        for key in tensors:
            if key.endswith(".mlp.router"):
                tensors[key] = (tensors[key].float() * 0.02).to(torch.bfloat16)
        write_safetensors(os.path.join(steady, "model.safetensors"), tensors)
        with open(os.path.join(steady, "config.json"), "w") as f:
            json.dump(raw, f)
        out[name, "bfloat16"] = steady
    return out


def read_tensors(folder):
    from tinyserve_llm_b200.weights.safetensors_io import SafetensorsFile
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    return {n: f.tensor(n) for n in f.names()}


def ids_of(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


_PLAIN = {}


def plain_logits(name, folder, ids):
    key = (folder, tuple(ids))
    if key not in _PLAIN:
        _PLAIN[key] = plain.forward(CONFIGS[name], read_tensors(folder), ids)
    return _PLAIN[key]


class Engine:
    """The engine's model, cache manager and step function on a small pool; logits are collected per request."""

    def __init__(self, folder, dtype, page=16, pages=24, slots=4, cuda_graphs=False):
        from tinyserve_llm_b200.engine.loading import build_cache, load_model
        from tinyserve_llm_b200.engine.step import StepRunner
        self.model = load_model(folder, dtype, "cuda")
        self.layout, self.manager, self.storage = build_cache(self.model, page, pages, caching=False, num_state_slots=slots)
        self.runner = StepRunner(self.model, self.manager, self.storage, cuda_graphs=cuda_graphs, sightings_before_capture=1)
        self.got = {}

    def step(self, parts, end=(), last_only=False):
        """parts: (request, its next tokens); the logits of every fed token (or of each request's last) are kept."""
        from tinyserve_llm_b200.engine.step import StepEntry
        entries = []
        for name, tokens in parts:
            if name in self.manager.seqs:
                self.manager.extend(name, tokens)
            else:
                assert self.manager.admit(name, tokens), f"{name} does not fit"
            entries.append(StepEntry(name, tokens, [len(tokens) - 1] if last_only else list(range(len(tokens)))))
        logits = self.runner.step(entries).cpu().double()
        at = 0
        for e in entries:
            self.manager.commit(e.seq_id, len(e.tokens))
            self.got.setdefault(e.seq_id, []).append(logits[at:at + len(e.want)])
            at += len(e.want)
        for name in end:
            self.manager.release(name)

    def logits(self, name):
        return torch.cat(self.got[name])

    def run(self, name, ids, sizes, end=True, last_only=False):
        pos, k = 0, 0
        while pos < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - pos)
            k += 1
            self.step([(name, ids[pos:pos + n])], end=[name] if end and pos + n == len(ids) else [], last_only=last_only)
            pos += n
        return self.logits(name)


def close(got, want, dtype):
    """
    float32: every position to rounding (the sharp comparison).  bfloat16: the error's root mean
    square against the logits' own spread.
    """
    if dtype == "float32":
        torch.testing.assert_close(got, want, atol=3e-4, rtol=1e-4)
    else:
        err = (got - want).pow(2).mean(-1).sqrt() / want.std()
        assert float(err.max()) < 0.12 and float(err.median()) < 0.04, \
            f"relative error: worst {float(err.max()):.3f} at {int(err.argmax())}, median {float(err.median()):.3f}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_equals_the_plain_model(folders, name, dtype):
    ids = ids_of(CONFIGS[name]["vocab"], 83, 1)
    got = Engine(folders[name, dtype], dtype).run("a", ids, [len(ids)])
    close(got, plain_logits(name, folders[name, dtype], ids), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "recurrent", "latent_only"])
def test_prompt_then_token_by_token_and_portions_of_many_sizes(folders, name, dtype):
    """The same logits whether the tokens come at once, one by one after a head, or in portions down to two tokens."""
    ids = ids_of(CONFIGS[name]["vocab"], 120, 2)
    want = plain_logits(name, folders[name, dtype], ids)
    decoded = Engine(folders[name, dtype], dtype).run("a", ids, [30] + [1] * 90)          # windows of 5, 21, 33, 50 pass over decoded tokens
    close(decoded, want, dtype)
    portions = Engine(folders[name, dtype], dtype).run("a", ids, [2, 3, 17, 2, 16, 5, 31, 1, 1, 2])
    close(portions, want, dtype)
    one_by_one = Engine(folders[name, dtype], dtype).run("a", ids[:40], [1])              # the first tokens, alone
    close(one_by_one, want[:40], dtype)
    if dtype == "float32":                                                           # the cut changes nothing beyond rounding
        torch.testing.assert_close(decoded, portions, atol=2e-5, rtol=1e-5)


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_requests_in_one_batch_and_reused_pages_and_slots(folders, dtype, graphs):
    """
    Five requests through three state slots and a pool that holds less than their sum: portions of
    some beside single tokens of others, requests that sit a step out, ended requests whose pages
    and slots the next ones take (a state that is not zeroed, or a page read through a stale table,
    shows).  With `graphs`, every step is replayed from a CUDA graph from its first sighting on.
    """
    name = "mixed"
    vocab = CONFIGS[name]["vocab"]
    reqs = {k: ids_of(vocab, n, 10 + i) for i, (k, n) in enumerate((("a", 70), ("b", 33), ("c", 9), ("d", 58), ("e", 41)))}
    eng = Engine(folders[name, dtype], dtype, page=16, pages=12, slots=3, cuda_graphs=graphs)
    eng.step([("a", reqs["a"][:40]), ("b", reqs["b"][:2])])
    eng.step([("a", reqs["a"][40:41]), ("b", reqs["b"][2:19]), ("c", reqs["c"][:9])], end=["c"])
    eng.step([("b", reqs["b"][19:20])])                                             # a sits this one out
    eng.step([("d", reqs["d"][:3]), ("a", reqs["a"][41:70]), ("b", reqs["b"][20:33])], end=["a", "b"])   # d takes c's slot
    eng.step([("d", reqs["d"][3:35]), ("e", reqs["e"][:1])])
    eng.step([("e", reqs["e"][1:2]), ("d", reqs["d"][35:36])])
    for i in range(36, 58):
        both = [("d", reqs["d"][i:i + 1])]
        j = 2 + (i - 36)
        if j < 41:
            both.append(("e", reqs["e"][j:j + 1]))
        eng.step(both, end=["d"] if i == 57 else [])
    eng.step([("e", reqs["e"][24:41])], end=["e"])
    assert eng.manager.stats().pages_in_use == 0 and eng.manager.free_state_slots() == 3
    if graphs:
        assert eng.runner.graph_replays > 20
    alone = {}
    for k, ids in reqs.items():
        close(eng.logits(k), plain_logits(name, folders[name, dtype], ids), dtype)
        alone[k] = Engine(folders[name, dtype], dtype, page=16, pages=12, slots=3).run(k, ids, [len(ids)])
        if dtype == "float32":
            torch.testing.assert_close(eng.logits(k), alone[k], atol=2e-5, rtol=1e-5)


def test_large_steps_on_the_library_grouped_product_also_from_a_graph(folders):
    """With many (token, expert) pairs the routed layers' bfloat16 products go to the library's grouped product: same logits."""
    name, dtype = "wide", "bfloat16"
    ids = ids_of(CONFIGS[name]["vocab"], 150, 7)
    eng = Engine(folders[name, dtype], dtype, page=16, pages=24, cuda_graphs=True)
    ops = eng.model.rt.ops
    old, ops.grouped_mm_min_pairs = ops.grouped_mm_min_pairs, 64
    try:
        before = ops.calls.get("library_grouped_mm", 0)
        got = eng.run("a", ids, [64, 40, 2, 44], last_only=True)                    # 128, 80, 4, 88 pairs
        assert ops.calls.get("library_grouped_mm", 0) > before and eng.runner.graph_replays >= 3
    finally:
        ops.grouped_mm_min_pairs = old
    close(got, plain_logits(name, folders[name, dtype], ids)[[63, 103, 105, 149]], dtype)


def test_decoding_with_the_keys_of_a_token_split_over_several_blocks(folders):
    """A decoded token far into a window of 300 keys: its keys are split over CTAs and merged; whole prompt and decode agree."""
    import copy
    from tinyserve_llm_b200.weights import write_random_model
    raw = copy.deepcopy(C.LATENT_ONLY)
    raw["layers"][0]["mixer"]["mask"]["size"] = 300
    raw["layers"][1]["mixer"]["mask"]["size"] = 1000
    folder = folders["latent_only", "float32"] + "_long_window"
    write_random_model(folder, raw, 77, **C.WEIGHTS)
    ids = ids_of(raw["vocab"], 420, 8)
    want = plain.forward(raw, read_tensors(folder), ids)
    for dtype in ("float32", "bfloat16"):
        eng = Engine(folder, dtype, page=16, pages=30)
        got = eng.run("a", ids, [390] + [1] * 30)
        assert eng.model.rt.ops.lib.ts_latent_attention_scratch_floats(1, 5, 40, 391) > 0     # the decoded tokens were split
        if dtype == "float32":
            torch.testing.assert_close(got, want, atol=3e-4, rtol=1e-4)
        else:
            err = (got - want).pow(2).mean(-1).sqrt() / want.std()
            assert float(err.median()) < 0.03 and float((err > 0.08).double().mean()) < 0.1    # routers as drawn: see `folders`


def test_long_decoding_keeps_its_state_and_gives_pages_back(folders):
    """300 tokens one by one through windows of 21 and 50 on pages of 16: the window groups' pools stay small."""
    name = "mixed"
    ids = ids_of(CONFIGS[name]["vocab"], 300, 3)
    dtype = "float32"
    eng = Engine(folders[name, dtype], "float32", page=16, pages=6)                        # 96 tokens of pages for 300 tokens
    got = eng.run("a", ids, [7] + [1] * 293)
    close(got, plain_logits(name, folders[name, dtype], ids), "float32")
    assert eng.manager.stats().window_releases > 20


# ---------------------------------------------------------------------------------------------- mechanisms alone
def _latent_case(dtype, page, window, positions_and_contexts, rank=24, rot=8, heads=3, special=None):
    """
    The latent attention kernel alone on a cache the test fills: returns (kernel output, plain output).
    `special` = (request, key position): that key's latent is made to dominate the scores of head 0,
    so whether it is seen decides the output.
    """
    from gpu_util import i32
    from types import SimpleNamespace
    from tinyserve_llm_b200.cache.storage import EntryBinding
    from tinyserve_llm_b200.ops import get_ops
    ops = get_ops()
    g = torch.Generator().manual_seed(5)
    width = rank + rot
    ctxs = [c for _, c in positions_and_contexts]
    pages_of = [-(-c // page) for c in ctxs]
    num_pages = sum(pages_of) + 2
    order = torch.randperm(num_pages, generator=g).tolist()                         # scattered pages
    tables, at = [], 0
    for n in pages_of:
        tables.append(order[at:at + n]); at += n
    pool = torch.full((num_pages, 1, 1, page, width), float("nan"), dtype=dtype, device="cuda")
    rows = [torch.randn(c, width, generator=g) * 0.5 for c in ctxs]
    if special is not None:
        s, j = special
        rows[s][j, :rank] = 0.0
        rows[s][j, 0] = 30.0
    for s, r in enumerate(rows):
        r = r.to(dtype)
        rows[s] = r.double()
        for j in range(r.shape[0]):
            pool[tables[s][j // page], 0, 0, j % page] = r[j].cuda()
    tw = max(len(t) for t in tables)
    table = i32([t + [-1] * (tw - len(t)) for t in tables])
    binding = EntryBinding(pool, None, page * width, 0, page, num_pages, table, tw, True)
    positions, seqs = [], []
    for s, (ps, _) in enumerate(positions_and_contexts):
        positions += ps; seqs += [s] * len(ps)
    T = len(positions)
    ctx = SimpleNamespace(positions=i32(positions), seq_of_token=i32(seqs))
    q_lat = torch.randn(T, heads, rank, generator=g)
    if special is not None:
        q_lat[:, 0, :] = 0.0
        q_lat[:, 0, 0] = 1.0
    q = (torch.randn(T, heads * (4 + rot), generator=g)).to(dtype)
    freq = torch.tensor([100.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32, device="cuda")
    scale = 0.4
    out = ops.latent_attention(q_lat.cuda(), q.cuda(), ctx, binding, heads, 4 + rot, 4, rank, rot, freq, scale, window)
    want = torch.zeros(T, heads, rank, dtype=torch.float64)
    qd = q.double().view(T, heads, 4 + rot)
    for t in range(T):
        s, p = seqs[t], positions[t]
        lo = max(0, p - window + 1) if window else 0
        keys = rows[s][lo:p + 1]
        q_rot = plain.rotate_half(qd[t:t + 1, :, 4:], torch.tensor([p]), rot, 100.0)[0]       # keys are stored rotated already
        sc = (torch.einsum("hd,jd->hj", q_lat[t].double(), keys[:, :rank]) + torch.einsum("hr,jr->hj", q_rot, keys[:, rank:])) * scale
        want[t] = torch.softmax(sc, -1) @ keys[:, :rank]
    return out.cpu().double(), want


@pytest.mark.parametrize("rank, rot", [(24, 8), (64, 16), (96, 32)])        # the second and third: sizes the tensor-core kernel takes
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attention_sees_exactly_its_window(dtype, rank, rot):
    """
    One key dominates head 0: queries whose window still holds it return its latent, the next query
    does not.  The key sits at a page's last slot and the queries come both as a prompt portion and
    as single tokens; another request in the batch has a different length.
    """
    page, window, key = 16, 37, 31                                                  # last slot of the second page
    inside, outside = key + window - 1, key + window                               # the last query that sees it, the first that does not
    cases = [(list(range(inside - 3, outside + 3)), outside + 3), ([outside], outside + 1), ([inside], inside + 1), ([4], 5)]
    got, want = _latent_case(dtype, page, window, cases, rank=rank, rot=rot, special=(0, key))
    tol = dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=0.04, rtol=0.02)
    torch.testing.assert_close(got, want, **tol)
    seen = got[:, 0, 0]                                                             # channel 0 of head 0: 30 if the key is seen
    assert all(float(v) > 25 for v in seen[:4]) and all(abs(float(v)) < 5 for v in seen[4:6])
    # the other requests hold their own caches: the dominant key is request 0's alone
    assert abs(float(seen[6])) < 5 and abs(float(seen[7])) < 5 and abs(float(seen[8])) < 5


@pytest.mark.parametrize("dtype, rank, rot, heads", [(torch.float32, 24, 8, 3), (torch.float32, 40, 4, 11), (torch.bfloat16, 64, 16, 3),
                                                     (torch.bfloat16, 128, 32, 19)])
def test_latent_attention_far_keys_without_a_window_and_first_tokens(dtype, rank, rot, heads):
    """
    No window: a key hundreds of positions back, among many, is found; position 0 sees itself only.  The
    step is small, so each token's keys are split over several CTAs and merged (19 heads: two groups of rows).
    """
    got, want = _latent_case(dtype, 16, 0, [([0, 1, 2, 499], 500), ([250], 251)], rank=rank, rot=rot, heads=heads, special=(0, 3))
    tol = dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=0.04, rtol=0.02)
    torch.testing.assert_close(got, want, **tol)
    assert float(got[3, 0, 0]) > 25 and abs(float(got[0, 0, 0])) < 5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["head", "channel_logits"])
def test_linear_recurrence_kernel(dtype, mode):
    """
    The recurrence kernel alone: two requests of unequal length in one launch, one continuing from a
    state an earlier launch left (cut at a place that is no multiple of the kernel's tile), sizes that
    are no multiples of the kernel's own (dim 20, vdim 37), rotation over part of a head, and a far
    token: with a decay close to one, the first token's value is still read 150 tokens later.
    """
    from gpu_util import i32
    from types import SimpleNamespace
    from tinyserve_llm_b200.cache.storage import EntryBinding
    from tinyserve_llm_b200.ops import get_ops
    ops = get_ops()
    g = torch.Generator().manual_seed(9)
    H, D, V, rot, tau = 3, 20, 37, 8, 4.0
    lens = [151, 23]
    T = sum(lens)
    y = (torch.randn(T, 2 * H * D + H * V + 5, generator=g) * 0.5).to(dtype)        # q | k | v in one row, as a projection leaves them
    y[0, H * D:2 * H * D] = 2.0                                                     # the first token's key ...
    y[150, :H * D] = 2.0                                                            # ... and the query that reads it back
    z = torch.randn(T, H * D, generator=g) + 6.0                                    # decays near one
    bias = torch.randn(H * D, generator=g) * 0.1
    decays = torch.tensor([0.999, 0.9, 0.5])
    freq_host = [50.0 ** (-2.0 * i / rot) for i in range(rot // 2)]
    position = SimpleNamespace(frequencies=torch.tensor(freq_host, dtype=torch.float32, device="cuda"), dims=rot)
    state = torch.zeros((4, H * D * V * 4 + 256), dtype=torch.uint8, device="cuda")
    yd = y.cuda()
    q, k, v = yd[:, :H * D], yd[:, H * D:2 * H * D], yd[:, 2 * H * D:2 * H * D + H * V]
    slots = [2, 0]

    def launch(ranges):
        """One launch over the given (begin, end) token ranges of the two requests."""
        rows = [r for s, (a, b) in enumerate(ranges) for r in range(sum(lens[:s]) + a, sum(lens[:s]) + b)]
        idx = torch.tensor(rows, device="cuda")
        pos = [p for (a, b) in ranges for p in range(a, b)]
        cu = [0]
        for a, b in ranges:
            cu.append(cu[-1] + b - a)
        sub = yd[idx].contiguous()
        ctx = SimpleNamespace(positions=i32(pos), cu_q=i32(cu))
        binding = EntryBinding(None, None, 0, 0, 16, 0, None, 0, True, -1, state[:, :H * D * V * 4], i32(slots))
        o = ops.linear_recurrence(sub[:, :H * D], sub[:, H * D:2 * H * D], sub[:, 2 * H * D:2 * H * D + H * V], ctx, binding,
                                  heads=H, dim=D, vdim=V, z=z.cuda()[idx].contiguous() if mode == "channel_logits" else None,
                                  bias=bias.cuda() if mode == "channel_logits" else None,
                                  head_decays=decays.cuda() if mode == "head" else None, inv_tau=1.0 / tau, q_scale=0.7,
                                  k_scale=1.3, position=position)
        return rows, o.cpu().double()

    got = torch.zeros(T, H * V, dtype=torch.float64)
    for ranges in ([(0, 37), (0, 2)], [(37, 151), (2, 23)]):                        # 37 and 2: not the kernel's tile of 16
        rows, o = launch(ranges)
        got[rows] = o
    want = torch.zeros(T, H, V, dtype=torch.float64)
    yy = y.double()
    at = 0
    for n in lens:
        pos = torch.arange(n)
        qq = plain.rotate_half(yy[at:at + n, :H * D].view(n, H, D), pos, rot, 50.0) * 0.7
        kk = plain.rotate_half(yy[at:at + n, H * D:2 * H * D].view(n, H, D), pos, rot, 50.0) * 1.3
        vv = yy[at:at + n, 2 * H * D:2 * H * D + H * V].view(n, H, V)
        if mode == "head":
            a = decays.double()[None, :, None].expand(n, H, D)
        else:
            a = torch.sigmoid(z[at:at + n].double() + bias.double()).pow(1.0 / tau).view(n, H, D)
        S = torch.zeros(H, D, V, dtype=torch.float64)
        for t in range(n):
            S = a[t][:, :, None] * S + kk[t][:, :, None] * vv[t][:, None, :]
            want[at + t] = torch.einsum("hdv,hd->hv", S, qq[t])
        at += n
    want = want.view(T, H * V)
    torch.testing.assert_close(got, want, atol=2e-4, rtol=2e-4)
    # the far token matters: without the first token's key the read-back at token 150 is another number
    assert float((want[150, :V] - want[149, :V]).abs().max()) > 1.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_stream_norm_kernel(dtype):
    from gpu_util import i32
    from tinyserve_llm_b200.ops import get_ops
    ops = get_ops()
    g = torch.Generator().manual_seed(3)
    T, W, eps = 7, 100, 1e-3
    stream = torch.randn(T, W, generator=g) * 3
    branch = (torch.randn(T, W, generator=g) * 5).to(dtype)
    wc, wo = 1 + torch.randn(W, generator=g) * 0.3, 1 + torch.randn(W, generator=g) * 0.3
    s = stream.cuda()
    out = ops.stream_norm(branch.cuda(), wc.cuda(), s, wo.cuda(), eps, dtype)
    want_s = stream.double() + plain.rms_unit(branch.double(), eps) * wc.double()
    torch.testing.assert_close(s.cpu().double(), want_s, atol=1e-5, rtol=1e-5)     # the stream stays float32 in both dtypes
    want = plain.rms_unit(want_s, eps) * wo.double()
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=0.02, rtol=0.01)
    torch.testing.assert_close(out.cpu().double(), want, **tol)
    rows = i32([5, 0])
    before = s.clone()
    picked = ops.stream_norm(branch.cuda(), wc.cuda(), s, wo.cuda(), eps, dtype, rows=rows)
    assert torch.equal(s, before)                                                   # with rows, the stream is read only
    want_rows = plain.rms_unit(want_s[[5, 0]] + plain.rms_unit(branch.double()[[5, 0]], eps) * wc.double(), eps) * wo.double()
    torch.testing.assert_close(picked.cpu().double(), want_rows, **tol)
    table = (torch.randn(11, W, generator=g)).to(dtype)
    ids = i32([3, 10, 0, 3, 7, 7, 1])
    fresh = torch.empty(T, W, device="cuda")
    out = ops.stream_norm(None, None, fresh, wo.cuda(), eps, dtype, table=table.cuda(), ids=ids, scale=2.5)
    rows_ = table.double()[ids.cpu().long()] * 2.5
    torch.testing.assert_close(fresh.cpu().double(), rows_, atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(out.cpu().double(), plain.rms_unit(rows_, eps) * wo.double(), **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts, top, shared", [(6, 3, True), (5, 1, False), (40, 4, True)])
def test_routed_experts_part(dtype, experts, top, shared):
    """The routed feed-forward alone, against the plain one; 50 tokens so that experts get unequal, ragged stretches."""
    from types import SimpleNamespace
    from tinyserve_llm_b200.config.spec import GatedMLPSpec, RoutedExpertsSpec
    from tinyserve_llm_b200.ops import get_ops
    from tinyserve_llm_b200.parts.base import Runtime, part_class
    from tinyserve_llm_b200.parts import model  # noqa: F401  (registers the parts)
    from tinyserve_llm_b200.weights import random_tensors
    width, ff = 48, 24
    e = GatedMLPSpec(hidden_size=width, intermediate_size=ff, activation="clamped_swish", limit=0.6, alpha=1.702,
                     tensor_names=("gate", "up", "down"))
    s = GatedMLPSpec(hidden_size=width, intermediate_size=40, activation="clamped_swish", limit=2.0, alpha=1.702,
                     tensor_names=("gate", "up", "down"))
    spec = RoutedExpertsSpec(hidden_size=width, num_experts=experts, top=top, expert=e, shared=s if shared else None)
    cls = part_class("feed_forward", spec)
    tensors = dict(random_tensors(cls.declare(spec), 17, std=0.3))
    tensors["router.b"] = tensors["router.b"] * 5                                   # the bias decides some choices
    rt = Runtime(dtype=dtype, device=torch.device("cuda", torch.cuda.current_device()), ops=get_ops())
    part = cls(spec, {k: v.cuda() for k, v in tensors.items()}, rt)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(50, width, generator=g).to(dtype)
    seq_of_token = torch.zeros(50, dtype=torch.int32, device="cuda")
    seq_of_token[-3:] = -1                                                          # padding rows of a replayed step
    got = part.forward(x.cuda(), SimpleNamespace(seq_of_token=seq_of_token)).cpu().double()[:47]
    f = {"router": {"experts": experts, "top": top}, "expert": {"limit": 0.6}, "shared": {"limit": 2.0} if shared else None}
    want = plain.ff_moe(f, {k: v.double() for k, v in tensors.items()}, x.double()[:47])
    tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else dict(atol=0.06, rtol=0.05)
    torch.testing.assert_close(got, want, **tol)


@pytest.mark.parametrize("rows", [1, 8, 100, 640])        # the weight-streaming kernel, the library + activation kernel, tcgen05
@pytest.mark.parametrize("activation, limit, alpha", [("relu", 0.0, 1.0), ("clamped_swish", 0.7, 1.702)])
def test_gated_products_with_the_activation_in_their_epilogue(rows, activation, limit, alpha):
    from tinyserve_llm_b200.ops import get_ops
    ops = get_ops()
    g = torch.Generator().manual_seed(rows)
    K, inter = 256, 200
    x = torch.randn(rows, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * inter, K, generator=g) * 0.08).to(torch.bfloat16)
    got = ops.linear_gated(x.cuda(), w.cuda(), activation, limit, alpha).cpu().double()
    y = x.double() @ w.double().T
    gate, up = y[:, :inter], y[:, inter:]
    if activation == "relu":
        want = torch.relu(gate) * up
    else:
        gate, up = gate.clamp(max=limit), up.clamp(-limit, limit)
        want = gate * torch.sigmoid(alpha * gate) * (up + 1.0)
    torch.testing.assert_close(got, want, atol=0.03, rtol=0.03)
    x32, w32 = x.float().cuda(), w.float().cuda()
    torch.testing.assert_close(ops.linear_gated(x32, w32, activation, limit, alpha).cpu().double(), want, atol=1e-4, rtol=1e-4)


def test_router_ties_go_to_the_lower_index_and_shares_are_a_softmax():
    from types import SimpleNamespace
    from tinyserve_llm_b200.ops import get_ops
    ops = get_ops()
    logits = torch.tensor([[0.0, 2.0, 2.0, -1.0, 2.0, 0.5], [5.0, 1.0, 0.0, 4.0, -3.0, 4.5]], device="cuda")
    chosen, share, offsets, pair_of_row, row_of_pair = ops.moe_route(logits, None, SimpleNamespace(), 2)
    assert chosen.tolist() == [[1, 2], [0, 5]]
    want = torch.softmax(torch.tensor([[2.0, 2.0], [5.0, 4.5]]), -1)
    torch.testing.assert_close(share.cpu(), want)
    assert offsets.tolist() == [0, 1, 2, 3, 3, 3, 4]
    assert sorted(pair_of_row.tolist()) == [0, 1, 2, 3] and [pair_of_row.tolist()[r] for r in row_of_pair.tolist()] == [0, 1, 2, 3]


# ---------------------------------------------------------------------------------------------- entry points
def test_replay_program_on_a_model_folder(folders, tmp_path):
    """bin/trace_run on a Duduvik folder: portions, a decoded tail, two requests side by side, a reused slot."""
    name = "wide"
    vocab = CONFIGS[name]["vocab"]
    a, b = ids_of(vocab, 90, 21), ids_of(vocab, 70, 22)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:64], "want": [0, 63]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[64:66], "want": [1]}, {"id": "b", "tokens": b[:69], "want": [68]}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[69:], "want": [0]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": a[66:], "want": [23]}], "end": ["a"]},
        {"step": 4, "entries": [{"id": "c", "tokens": b, "want": [69]}], "end": ["c"]},
    ]
    rows = {0: [("a", 0), ("a", 63)], 1: [("a", 65), ("b", 68)], 2: [("b", 69)], 3: [("a", 89)], 4: [("b", 69)]}
    for dtype in ("float32", "bfloat16"):
        want = {"a": plain_logits(name, folders[name, dtype], a), "b": plain_logits(name, folders[name, dtype], b)}
        out = tmp_path / dtype
        proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folders[name, dtype], "--dtype", dtype,
                               "--out", str(out), "--max-tokens", "256", "--max-requests", "2"],
                              input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
        assert [line for line in proc.stdout.splitlines() if line.startswith("done")] == [f"done {i}" for i in range(5)]
        got, expected = [], []
        for step, places in rows.items():
            got.append(torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(places), vocab)).double())
            expected += [want[r][p] for r, p in places]
        close(torch.cat(got), torch.stack(expected), dtype)


@pytest.mark.parametrize("name", ["mixed", "recurrent"])
def test_greedy_generation_through_the_entry_point(folders, name):
    """LLM.generate with the scheduler, prompt portions, CUDA graphs and running ahead: the plain model's greedy tokens."""
    from tinyserve_llm_b200 import LLM, CacheConfig, SamplingParams, SchedulerConfig
    raw, dtype = CONFIGS[name], "float32"
    tensors = read_tensors(folders[name, dtype])
    prompts = [ids_of(raw["vocab"], n, 30 + n) for n in (3, 41, 18, 77, 1)]
    new = 12
    want = []
    for p in prompts:
        ids = list(p)
        for _ in range(new):
            ids.append(int(plain.forward(raw, tensors, ids)[-1].argmax()))
        want.append(ids[len(p):])
    llm = LLM(folders[name, dtype], SchedulerConfig(max_model_len=128, max_num_seqs=3, max_num_batched_tokens=48, prefill_chunk=20),
              CacheConfig(block_size=16), dtype="float32", num_blocks=24, seed=0)
    done = llm.generate(prompts, SamplingParams(max_tokens=new, temperature=0.0, ignore_eos=True))
    assert [c.token_ids[0] for c in done] == want
