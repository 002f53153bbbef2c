"""The Zulozen decoder on the device against the plain implementation (tests/plain_zulozen.py): whole prompts,
decoding through the cache, portions down to two tokens, unequal batches against each sequence alone, slots and
pages used again, long decoding over several blocks of positions, greedy generation through the library's entry
point, the trace runner, and the kernels of each mechanism alone with inputs made so that a block's edge, a far
key, the sink or a first token shows."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_zulozen as pz
from zulozen_models import CONFIGS, as_float64, write_model
import helpers
from helpers import assert_same_engine, tokens

pytestmark = pytest.mark.gpu

SEEDS = {"mixed": 21, "odd": 22, "wide": 23, "open": 24, "all_experts": 25}
LENGTHS = {"mixed": 150, "odd": 141, "wide": 270, "open": 90, "all_experts": 330}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        d = str(tmp_path_factory.mktemp("zulozen_" + name))
        out[name] = (d, as_float64(write_model(d, cfg, SEEDS[name])))
    return out


_models: dict = {}


def model(folders, name, dtype):
    import camelid_b200
    if (name, dtype) not in _models:
        _models[(name, dtype)] = camelid_b200.load(folders[name][0], dtype=dtype)
    return _models[(name, dtype)]


_plain: dict = {}


def plain(folders, name, ids):
    """(logits float64 [tokens, vocab], per row the smallest margin of a router's choice over all routed layers)."""
    key = (name, tuple(ids))
    if key not in _plain:
        margins = []
        logits = pz.forward(CONFIGS[name], folders[name][1], list(ids), margins=margins)
        margin = np.min(np.stack(margins), axis=0) if margins else np.full(len(ids), np.inf)
        _plain[key] = (torch.from_numpy(logits), margin)
    return _plain[key]


def assert_close(got, ref_and_margin, dtype, what=""):
    """The library's tolerances. In float32 every row counts. In bfloat16 the router scores rows that carry the
    rounding of everything before them, so a near tie may fall the other way; the row then goes through another
    expert, and every later row that attends to it moves too. So the bound on single rows is asked of the rows
    before the first near tie of the sequence, and of all rows together that most of them keep it."""
    ref, margin = ref_and_margin
    got = torch.as_tensor(got)
    if dtype == "bfloat16" and np.isinf(margin).all():          # no choice to make anywhere: every row counts
        return helpers.assert_close(got, ref, dtype, what)
    if dtype == "bfloat16":
        clear = np.minimum.accumulate(margin) > 0.05
        rows = helpers.row_errors(got, ref)
        assert float(rows.median()) <= helpers.TOL[dtype], f"{what}: the median row is off by {float(rows.median()):.3e}"
        n = int(clear.sum())
        if n == 0:
            return
        got, ref = got[:n], ref[:n]
    helpers.assert_close(got, ref, dtype, what)


def run_cut(lm, cache, ids, cut):
    """Feed ``ids`` in portions of the sizes ``cut`` (the rest one by one); logits of every position."""
    from camelid_b200.engine.model import StepEntry
    slot = cache.alloc_slot()
    out, at = [], 0
    sizes = list(cut) + [1] * (len(ids) - sum(cut))
    for n in sizes:
        out.append(lm.step(cache, [StepEntry(slot, ids[at:at + n], list(range(n)))]).cpu())
        at += n
    cache.free_slot(slot)
    return torch.cat(out)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt_and_decoding_match_plain(cuda, folders, name, dtype):
    lm = model(folders, name, dtype)
    ids = tokens(SEEDS[name], LENGTHS[name], CONFIGS[name]["vocab"])
    ref = plain(folders, name, ids)
    cache = lm.new_cache(1024)
    whole = run_cut(lm, cache, ids, [len(ids)])
    assert_close(whole, ref, dtype, f"{name} whole prompt")
    n = len(ids)
    decoded = run_cut(lm, cache, ids, [n - 40])                # the last tokens one by one (captured steps)
    assert_close(decoded, ref, dtype, f"{name} decoded")
    if dtype == "float32":
        assert_same_engine(whole, decoded, f"{name} whole against decoded", tol=1e-5)
    lm.model.check_device_errors()
    cache.book.audit()


@pytest.mark.parametrize("name,cut", [("mixed", [7, 2, 3, 2, 50, 1, 1, 2, 64, 2]), ("odd", [64, 2, 63, 1, 2, 5]),
                                      ("open", [1, 2, 2, 3, 70]), ("wide", [2, 126, 2, 3, 128, 2])])
def test_portions_of_a_prompt(cuda, folders, name, cut):
    lm = model(folders, name, "float32")
    ids = tokens(SEEDS[name], LENGTHS[name], CONFIGS[name]["vocab"])
    cache = lm.new_cache(1024)
    got = run_cut(lm, cache, ids, cut)
    assert_close(got, plain(folders, name, ids), "float32", f"{name} in portions {cut}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "odd", "wide"])
def test_unequal_batch_against_each_alone(cuda, folders, name, dtype):
    """Prompts of 1, 17 and 135 tokens start together, are decoded together and end one after the other."""
    from camelid_b200.engine.model import StepEntry
    lm = model(folders, name, dtype)
    vocab = CONFIGS[name]["vocab"]
    seqs = [tokens(100 + i, n, vocab) for i, n in enumerate((9, 30, 150))]
    prompt = [1, 17, 135]
    cache = lm.new_cache(1024)
    slots = [cache.alloc_slot() for _ in seqs]
    got = [[] for _ in seqs]
    logits = lm.step(cache, [StepEntry(s, q[:p], list(range(p))) for s, q, p in zip(slots, seqs, prompt)]).cpu()
    at = 0
    for i, p in enumerate(prompt):
        got[i].append(logits[at:at + p])
        at += p
    done = list(prompt)
    live = [0, 1, 2]
    while live:
        logits = lm.step(cache, [StepEntry(slots[i], [seqs[i][done[i]]], [0]) for i in live]).cpu()
        for j, i in enumerate(live):
            got[i].append(logits[j:j + 1])
            done[i] += 1
        for i in [i for i in live if done[i] == len(seqs[i])]:
            cache.free_slot(slots[i])
        live = [i for i in live if done[i] < len(seqs[i])]
    for i, q in enumerate(seqs):
        assert_close(torch.cat(got[i]), plain(folders, name, q), dtype, f"{name} sequence {i} of a batch")
    cache.book.audit()


def test_slots_and_pages_used_again(cuda, folders):
    """A cache of three pages and one slot: every sequence gets the slot and the pages the one before gave back; the
    layers that see blocks of positions give their old pages back on the way, the layer that sees everything keeps them."""
    lm = model(folders, "open", "float32")
    cache = lm.new_cache(192, max_slots=1)
    for i, n in enumerate((130, 75, 190)):
        ids = tokens(200 + i, n, CONFIGS["open"]["vocab"])
        got = run_cut(lm, cache, ids, [n - 10])
        assert_close(got, plain(folders, "open", ids), "float32", f"sequence {i} in a slot used before")
        cache.book.audit()
    assert cache.book.slots.n_free == 1 and all(p.n_free == p.n for p in cache.book.pools)


def test_long_decoding_over_many_blocks(cuda, folders):
    lm = model(folders, "mixed", "float32")
    ids = tokens(5, 300, CONFIGS["mixed"]["vocab"])
    cache = lm.new_cache(512)
    got = run_cut(lm, cache, ids, [3])
    assert_close(got, plain(folders, "mixed", ids), "float32", "297 tokens decoded one by one")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(cuda, folders, dtype):
    """``generate`` (scheduler, batches, the decode loop on the device) picks the plain implementation's tokens."""
    lm = model(folders, "mixed", dtype)
    cfg = CONFIGS["mixed"]
    prompts = [tokens(300, 5, cfg["vocab"]), tokens(301, 19, cfg["vocab"]), tokens(302, 1, cfg["vocab"])]
    for _ in range(2):                                         # the second call uses the slots again
        out = lm.generate(prompts, max_tokens=12)
        for p, new in zip(prompts, out):
            assert len(new) == 12
            seq = list(p)
            for tok in new:
                ref, margin = plain(folders, "mixed", seq)
                top2 = torch.topk(ref[-1], 2).values
                if dtype == "float32" or (float(top2[0] - top2[1]) > 0.25 and margin.min() > 0.3):
                    assert tok == int(ref[-1].argmax()), (seq, new)
                seq.append(tok)


def test_weights_drawn_on_the_device_match_the_folder(cuda, tmp_path):
    """``from_random`` (what the benchmark uses) and a folder written on the host hold the same model."""
    import camelid_b200
    from camelid_b200.weights.random_init import write_random_model
    cfg = CONFIGS["mixed"]
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=5)
    a = camelid_b200.load(folder, dtype="bfloat16")
    b = camelid_b200.from_random(cfg, seed=5, dtype="bfloat16")
    prompts = [tokens(1, 12, cfg["vocab"]), tokens(2, 3, cfg["vocab"])]
    assert a.generate(prompts, max_tokens=6) == b.generate(prompts, max_tokens=6)


def test_trace_runner_replays_a_zulozen_model(cuda, folders, tmp_path):
    folder, _ = folders["odd"]
    cfg = CONFIGS["odd"]
    a, b = tokens(1, 40, cfg["vocab"]), tokens(2, 4, cfg["vocab"])
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:38], "want": [0, 32, 33, 37]}, {"id": "b", "tokens": b[:1], "want": [0]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[38:39], "want": []}, {"id": "b", "tokens": b[1:2], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[39:40], "want": [0]}, {"id": "b", "tokens": b[2:3], "want": [0]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": b[3:4], "want": [0]}], "end": ["b"]}]
    exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "trace_run")
    r = subprocess.run([sys.executable, exe, "--model", folder, "--dtype", "float32", "--out", str(tmp_path), "--max-tokens", "128"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == [f"done {i}" for i in range(4)]
    ra, rb = plain(folders, "odd", a)[0], plain(folders, "odd", b)[0]
    want = {0: torch.stack([ra[0], ra[32], ra[33], ra[37], rb[0]]), 1: rb[1:2], 2: torch.stack([ra[39], rb[2]]), 3: rb[3:4]}
    for i, ref in want.items():
        got = torch.from_numpy(np.fromfile(tmp_path / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"]))
        helpers.assert_close(got, ref, "float32", f"step {i}")


# ---- each mechanism's kernels alone -------------------------------------------------------------

def arrays(cuda, starts, news):
    """The packed-row arrays of a step: one slot per sequence, slot = its index."""
    row_seq = np.repeat(np.arange(len(news)), news)
    row_pos = np.concatenate([np.arange(s, s + n) for s, n in zip(starts, news)])
    dev = lambda a: torch.as_tensor(np.asarray(a), dtype=torch.int32, device=cuda)      # noqa: E731
    return {"row_seq": dev(row_seq), "row_pos": dev(row_pos)}


def portions(n, cut):
    sizes = list(cut) + [1] * (n - sum(cut))
    at = 0
    for s in sizes:
        yield at, s
        at += s


def _paged(cuda, T, G, D, Dv, dtype):
    pages = (T + 63) // 64
    order = list(range(pages))[::-1]                                   # pages in another order than positions
    table = torch.tensor([order + [-1]], dtype=torch.int32, device=cuda)
    k = torch.full((pages + 1, G, 64, D), float("nan"), dtype=dtype, device=cuda)
    v = torch.full((pages + 1, G, 64, Dv), float("nan"), dtype=dtype, device=cuda)
    return table, k, v


@pytest.mark.parametrize("cut", [[640], [100, 2, 60, 300, 2], [5]])
@pytest.mark.parametrize("block", [70, 600])
def test_attention_kernels_at_a_blocks_edge_and_far_back(cuda, cut, block):
    """Keys that every query loves stand at the first position, at the edges of cache pages and of blocks of positions:
    a query's output jumps when it crosses into the next block and loses them. With blocks of 600 positions a loved
    key at position 2 is still found by position 599, among hundreds of others, and is gone at 600. The sink takes a
    known share; the gate is one number per head; q and k are normed over all heads at once and rotated in pairs of
    neighbours. Keys and values of different sizes, 3 query heads per kv head."""
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(1)
    T, H, G, D, Dv, scale, rot, base, eps = 640, 6, 2, 24, 40, 0.5, 8, 50.0, 1e-5
    q = torch.randn(T, H * D, generator=gen) * 0.3
    k = torch.randn(T, G * D, generator=gen) * 0.3
    v = torch.randn(T, G, Dv, generator=gen)
    loved = (0, 2, 63, 64, 69, 70, 139, 140, 599, 600)
    for j in loved:                                                    # a channel outside the rotated ones stands out
        k[j] = 0.0
        k[j, [D - 1, 2 * D - 1]] = 6.0
    q.view(T, H, D)[:, :, D - 1] = 2.0
    qw, kw = 1.0 + 0.3 * torch.randn(H * D, generator=gen), 1.0 + 0.3 * torch.randn(G * D, generator=gen)
    qw.view(H, D)[:, D - 1], kw.view(G, D)[:, D - 1] = 1.0, 1.0
    sink = torch.tensor([-30.0, 0.0, 3.0, 6.0, 1.0, -2.0])
    gate = torch.randn(T, H, generator=gen)
    t = {"q": np.eye(H * D), "k": np.eye(G * D), "v": np.eye(G * Dv), "q.norm": qw.double().numpy(), "k.norm": kw.double().numpy()}
    cfg = {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "rot": {"dims": rot, "base": base}}
    # the plain projection with identity matrices: h carries q, k, v side by side
    qn = pz.rotate_interleaved(pz.rms_norm(q.double().numpy(), t["q.norm"], eps).reshape(T, H, D), np.arange(T), rot, base)
    kn = pz.rotate_interleaved(pz.rms_norm(k.double().numpy(), t["k.norm"], eps).reshape(T, G, D), np.arange(T), rot, base)
    ref = pz.attend(qn, kn, v.double().numpy(), scale, block, sink.double().numpy(), 1 / (1 + np.exp(-gate.double().numpy())))
    ref = torch.from_numpy(ref.reshape(T, H * Dv))
    edge = block if block < T else 0
    if edge:                                                           # the row that opens a block sees only itself
        assert float((ref[edge - 1] - ref[edge]).abs().max()) > 0.05
    proj = torch.cat([q, k, v.reshape(T, -1), gate], 1).to(cuda)
    inv_freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32, device=cuda)
    table, kp, vp = _paged(cuda, T, G, D, Dv, torch.float32)
    got = []
    for at, n in portions(T, cut):
        a = arrays(cuda, [at], [n])
        qo = torch.empty(n, H * D, device=cuda)
        ops.qkv_prepare(proj[at:at + n], qw.to(cuda), kw.to(cuda), 2, eps, inv_freq, rot, True, a["row_seq"], a["row_pos"], table,
                        qo, kp, vp, H, G, D, Dv)
        out = torch.empty(n, H * Dv, device=cuda)
        ops.window_attention(qo, kp, vp, table, a["row_seq"], a["row_pos"], None, None, proj[at:at + n], H * D + G * D + G * Dv,
                             out, H, G, D, Dv, 0, scale, chunk=block, sink=sink.to(cuda), gate_per_head=True)
        got.append(out.cpu())
    got = torch.cat(got).double()
    assert torch.isfinite(got).all()
    assert float((got - ref).abs().max()) < 2e-5 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("D,group,block", [(64, 3, 70), (128, 2, 200), (128, 1, 33), (64, 4, 1000)])
def test_prompt_attention_on_tensor_cores_with_blocks_sink_and_gate(cuda, D, group, block):
    """bfloat16 prompts with keys and values of 64 or 128 channels take the tcgen05 kernel: two sequences in one step, the
    first a portion that starts at position 150 of its sequence (blocks are counted from position 0, not from the cut),
    against the plain formula on the same bfloat16 q, k, v; a loved key just before a block's edge shows the edge."""
    from camelid_b200.csrc import ops
    from camelid_b200.parts import linear
    gen = torch.Generator().manual_seed(7)
    G, lens, starts = 2, [380, 67], [150, 0]
    H = G * group
    scale = D ** -0.5
    tile_rows, hpc, chunks = ops.attn_tc_tiling(H, G)
    sink = torch.randn(H, generator=gen) * 2
    total = [s + n for s, n in zip(starts, lens)]
    qs = [torch.randn(t, H, D, generator=gen).to(torch.bfloat16) for t in total]
    ks = [torch.randn(t, G, D, generator=gen).to(torch.bfloat16) for t in total]
    vs = [torch.randn(t, G, D, generator=gen).to(torch.bfloat16) for t in total]
    edge = (total[0] // block) * block - 1 if block < total[0] else 5
    ks[0][edge] = 0
    ks[0][edge, :, 0] = 30.0
    qs[0][:, :, 0] = 2.0
    gates = [torch.randn(t, H, generator=gen) for t in total]
    ref = torch.cat([torch.from_numpy(pz.attend(q.double().numpy(), k.double().numpy(), v.double().numpy(), scale, block,
                                                sink.double().numpy(), 1 / (1 + np.exp(-g.double().numpy())))).reshape(t, H * D)[st:]
                     for q, k, v, g, t, st in zip(qs, ks, vs, gates, total, starts)])
    pages = [(t + 63) // 64 for t in total]
    table = torch.full((2, max(pages)), -1, dtype=torch.int32)
    table[0, :pages[0]] = torch.arange(pages[0]) + pages[1]
    table[1, :pages[1]] = torch.arange(pages[1])
    table = table.to(cuda)
    kp = torch.zeros(sum(pages), G, 64, D, dtype=torch.bfloat16, device=cuda)
    vp = torch.zeros_like(kp)
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device=cuda)      # noqa: E731
    # the earlier part of the first sequence is in the cache already; then the step's rows
    n0 = starts[0]
    early = arrays(cuda, [0], [n0])
    proj = torch.cat([qs[0][:n0].reshape(n0, -1), ks[0][:n0].reshape(n0, -1), vs[0][:n0].reshape(n0, -1)], 1).float().to(cuda)
    ops.qk_norm_kv_write(proj, None, None, 1e-6, early["row_seq"], early["row_pos"], table,
                         torch.empty(n0, H * D, dtype=torch.bfloat16, device=cuda), kp, vp, H, G, D, D)
    a = arrays(cuda, starts, lens)
    rows = sum(lens)
    cat = lambda xs: torch.cat([x[st:].reshape(t - st, -1) for x, t, st in zip(xs, total, starts)])      # noqa: E731
    proj = torch.cat([cat(qs), cat(ks), cat(vs)], 1).float().to(cuda)
    gate = cat(gates).to(cuda)
    qn = torch.empty(rows, H * D, dtype=torch.bfloat16, device=cuda)
    ops.qk_norm_kv_write(proj, None, None, 1e-6, a["row_seq"], a["row_pos"], table, qn, kp, vp, H, G, D, D)
    tile_seq = [s for s, n in enumerate(lens) for _ in range(0, n, tile_rows)]
    tile_q0 = [q0 for n in lens for q0 in range(0, n, tile_rows)]
    row0 = [0, lens[0]]
    out = torch.empty(rows, H * D, dtype=torch.bfloat16, device=cuda)
    assert ops.attn_tc_usable(qn, out, D)
    ops.attn_prefill_tc(qn, out, kp, vp, table, dev(tile_seq), dev(tile_q0), len(tile_seq), dev(row0), dev(starts), dev(lens),
                        H, G, D, tile_rows, hpc, chunks, 0, scale, linear._err_word(cuda), None, None, block, sink.to(cuda), gate, 0)
    plain_kernel = torch.empty_like(out)
    ops.window_attention(qn, kp, vp, table, a["row_seq"], a["row_pos"], None, None, gate, 0, plain_kernel, H, G, D, D, 0, scale,
                         chunk=block, sink=sink.to(cuda), gate_per_head=True)
    linear.check_errors()
    for got, what in ((out, "tensor cores"), (plain_kernel, "plain kernel")):
        err = float((got.cpu().double() - ref).abs().max())
        assert err < 3e-2, f"{what}: {err}"


@pytest.mark.parametrize("norm_mode,interleaved,D,rot,splits", [(1, False, 12, 8, 1), (0, True, 16, 16, 3), (1, True, 7, 4, 2),
                                                                 (2, False, 24, 24, 11), (0, False, 8, 0, 1)])
def test_preparation_kernel_in_every_mode(cuda, norm_mode, interleaved, D, rot, splits):
    """Norm per head, over the whole projection or none; pairs of neighbours or of halves; an odd head size; the input
    as split sums; the gate's logits handed on."""
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(9)
    T, H, G, Dv, eps, base, extra = 70, 3, 1, 5, 1e-5, 100.0, 3
    n = H * D + G * D + G * Dv + extra
    parts = torch.randn(splits, T, n, generator=gen)
    x = parts.double().sum(0).numpy()
    wq = (1 + 0.3 * torch.randn(H * D if norm_mode == 2 else D, generator=gen))
    wk = (1 + 0.3 * torch.randn(G * D if norm_mode == 2 else D, generator=gen))
    q, k = x[:, :H * D], x[:, H * D:(H + G) * D]
    if norm_mode == 2:
        q, k = pz.rms_norm(q, wq.double().numpy(), eps), pz.rms_norm(k, wk.double().numpy(), eps)
    q, k = q.reshape(T, H, D), k.reshape(T, G, D)
    if norm_mode == 1:
        q, k = pz.rms_norm(q, wq.double().numpy(), eps), pz.rms_norm(k, wk.double().numpy(), eps)
    pos = np.arange(T)

    def turn(t):
        if not rot:
            return t
        if interleaved:
            return pz.rotate_interleaved(t, pos, rot, base)
        out, half = t.copy(), rot // 2
        ang = pos[:, None] * base ** (-2.0 * np.arange(half) / rot)[None, :]
        c, sn = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
        out[..., :half] = t[..., :half] * c - t[..., half:rot] * sn
        out[..., half:rot] = t[..., half:rot] * c + t[..., :half] * sn
        return out
    q, k = turn(q), turn(k)
    inv_freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32, device=cuda)
    table, kp, vp = _paged(cuda, T, G, D, Dv, torch.float32)
    a = arrays(cuda, [0], [T])
    qo, gate = torch.empty(T, H * D, device=cuda), torch.empty(T, extra, device=cuda)
    ops.qkv_prepare(parts.to(cuda), wq.to(cuda) if norm_mode else None, wk.to(cuda) if norm_mode else None, norm_mode, eps, inv_freq,
                    rot, interleaved, a["row_seq"], a["row_pos"], table, qo, kp, vp, H, G, D, Dv, gate)
    assert np.allclose(qo.cpu().double().numpy(), q.reshape(T, -1), atol=2e-5)
    assert np.allclose(gate.cpu().double().numpy(), x[:, -extra:], atol=2e-5)
    tb = table.cpu()[0]
    for t in (0, 63, 64, T - 1):
        assert np.allclose(kp[tb[t // 64], :, t % 64].cpu().double().numpy(), k[t], atol=2e-5)
        assert np.allclose(vp[tb[t // 64], :, t % 64].cpu().double().numpy(), x[t, (H + G) * D:(H + G) * D + G * Dv].reshape(G, Dv), atol=2e-5)


def test_sink_alone_takes_its_share(cuda):
    """One key of score zero and a sink of ln 3: the key's value comes out at a quarter."""
    from camelid_b200.csrc import ops
    D = Dv = 16
    table, kp, vp = _paged(cuda, 1, 1, D, Dv, torch.float32)
    kp.zero_()
    vp.fill_(8.0)
    a = arrays(cuda, [0], [1])
    out = torch.empty(1, Dv, device=cuda)
    ops.window_attention(torch.zeros(1, D, device=cuda), kp, vp, table, a["row_seq"], a["row_pos"], None, None, None, 0, out,
                         1, 1, D, Dv, 0, 1.0, chunk=4, sink=torch.tensor([float(np.log(3.0))], device=cuda))
    assert torch.allclose(out.cpu(), torch.full((1, Dv), 2.0), atol=1e-6)


@pytest.mark.parametrize("rows,E,top,ff", [(1, 5, 2, 24), (7, 3, 3, 16), (300, 5, 2, 48), (150, 16, 1, 8), (700, 3, 2, 272)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_routed_experts_kernels(cuda, rows, E, top, ff, dtype):
    """Routing, ordering by expert, the grouped products and the sum against the plain routed feed-forward: experts with
    no row, with one row, and (300 rows over 5 experts) with more rows than a tile; ties in the router go to the lower index."""
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(3)
    W = 48
    x = torch.randn(rows, W, generator=gen).to(dtype)
    t = {"router": torch.randn(E, W, generator=gen) * 0.5}
    for e in range(E):
        t[f"e{e}.gate"], t[f"e{e}.up"] = torch.randn(ff, W, generator=gen) * 0.2, torch.randn(ff, W, generator=gen) * 0.2
        t[f"e{e}.down"] = torch.randn(W, ff, generator=gen) * 0.2
    t = {n: w.to(dtype) for n, w in t.items()}
    t["router"] = t["router"].float()
    tn = {n: w.double().numpy() for n, w in t.items()}
    logits = x.float() @ t["router"].T
    if E == 16:
        logits[:, 5:] = logits[:, 4:5]                                  # experts 4..15 tie everywhere: the lowest wins, 5.. get no row
        tn["router"] = None
    logits = logits.to(cuda).contiguous()
    pairs = rows * top
    i32 = lambda n: torch.empty(n, dtype=torch.int32, device=cuda)      # noqa: E731
    ids, wts = i32(pairs), torch.empty(pairs, device=cuda)
    ops.route_topk(logits, top, False, False, ids, wts)
    score = torch.sigmoid(logits.double().cpu())
    want_ids = torch.argsort(-score, dim=1, stable=True)[:, :top]
    # the plain routed feed-forward on a router that reproduces these logits exactly: identity on the logits as inputs
    ref = torch.zeros(rows, W, dtype=torch.float64)
    for r in range(rows):
        for e in want_ids[r].tolist():
            ref[r] += torch.from_numpy(pz.gated_expert(float(score[r, e]) * x[r:r + 1].double().numpy(), tn, f"e{e}")[0])
    assert torch.equal(ids.cpu().view(rows, top).long(), want_ids)
    rank, counts, offsets, tiles, place = i32(pairs), i32(E), i32(E + 1), i32(E + 1), i32(pairs)
    ops.expert_plan(ids, E, rank, counts, offsets, tiles)
    assert counts.cpu().tolist() == torch.bincount(want_ids.reshape(-1), minlength=E).tolist() and int(offsets[E]) == pairs
    xd = x.to(cuda)
    xs = torch.empty(pairs, W, dtype=dtype, device=cuda)
    ops.expert_gather(xd, ids, wts, rank, offsets, top, True, xs, place)
    assert sorted(place.cpu().tolist()) == list(range(pairs))
    stack = lambda n: torch.stack([t[f"e{e}.{n}"] for e in range(E)]).to(cuda).contiguous()      # noqa: E731
    act = torch.empty(pairs, ff, dtype=dtype, device=cuda)
    ops.expert_gemm(xs, stack("gate"), stack("up"), act, offsets, tiles)
    ys = torch.empty(pairs, W, device=cuda)
    ops.expert_gemm(act, stack("down"), None, ys, offsets, tiles)
    out = torch.empty(rows, W, device=cuda)
    ops.expert_combine(ys, place, wts, top, False, None, out)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert float((out.double().cpu() - ref).abs().max()) < tol * max(1.0, float(ref.abs().max()))
    if dtype == torch.bfloat16 and ff % 16 == 0:
        # the same through the grouped product on the tensor cores (stretches cut into tiles of 128 rows)
        from camelid_b200.parts import linear
        ops.expert_plan(ids, E, rank, counts, offsets, tiles, ops.EXPERT_TILE_ROWS_TC)
        packed = torch.stack([linear.pack_gate_up(t[f"e{e}.gate"], t[f"e{e}.up"], 16) for e in range(E)]).to(cuda).contiguous()
        err = torch.zeros(1, dtype=torch.int32, device=cuda)
        act2, ys2 = torch.full_like(act, float("nan")), torch.full_like(ys, float("nan"))
        ops.gemm_tc_grouped(xs, packed, act2, ops.TC_SWIGLU, offsets, tiles, err)
        ops.gemm_tc_grouped(act2, stack("down"), ys2, ops.TC_STORE_F32, offsets, tiles, err)
        ops.expert_combine(ys2, place, wts, top, False, None, out)
        assert int(err.item()) == 0
        assert float((out.double().cpu() - ref).abs().max()) < tol * max(1.0, float(ref.abs().max()))


def test_dense_feed_forward_and_the_norm_behind_it(cuda):
    """act(x Wu^T + bu) with the squared ReLU from split sums and in place, and stream += m * rmsnorm(y + bias) * w."""
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(4)
    rows, W, F = 5, 40, 24
    part = torch.randn(3, rows, F, generator=gen)
    bias = torch.randn(F, generator=gen)
    ref = torch.clamp(part.double().sum(0) + bias.double(), min=0) ** 2
    out = torch.empty(rows, F, device=cuda)
    ops.act_from_partials(part.to(cuda), out, act=ops.ACT_RELU_SQUARED, bias=bias.to(cuda))
    assert torch.allclose(out.cpu().double(), ref, atol=1e-5)
    whole = part.sum(0).to(cuda).contiguous()
    ops.bias_act_(whole, bias.to(cuda), ops.ACT_RELU_SQUARED)
    assert torch.allclose(whole.cpu().double(), ref, atol=1e-5)
    y, b, w = torch.randn(2, rows, W, generator=gen), torch.randn(W, generator=gen), 1 + 0.3 * torch.randn(W, generator=gen)
    stream = torch.randn(rows, W, generator=gen)
    want = stream.double() + 0.35 * torch.from_numpy(pz.rms_norm((y.double().sum(0) + b.double()).numpy(), w.double().numpy(), 1e-5))
    s = stream.to(cuda)
    ops.norm_combine([(y.to(cuda), w.to(cuda))], s, 1e-5, 0.35, [b.to(cuda)])
    assert torch.allclose(s.cpu().double(), want, atol=1e-5)
    # the same in one pass with the norm that follows; a width that allows no 16-byte pieces too
    for width in (W, W - 3):
        w2 = 1 + 0.3 * torch.randn(width, generator=gen)
        yy, bb, ww, st = y[:, :, :width].contiguous(), b[:width].contiguous(), w[:width].contiguous(), stream[:, :width].contiguous()
        want = st.double() + 0.35 * torch.from_numpy(pz.rms_norm((yy.double().sum(0) + bb.double()).numpy(), ww.double().numpy(), 1e-5))
        want_x = torch.from_numpy(pz.rms_norm(want.numpy(), w2.double().numpy(), 2e-5))
        s2, x = st.to(cuda), torch.empty(rows, width, device=cuda)
        ops.post_norm_add(yy.to(cuda), bb.to(cuda), ww.to(cuda), 1e-5, 0.35, s2, w2.to(cuda), 2e-5, x)
        assert torch.allclose(s2.cpu().double(), want, atol=1e-5) and torch.allclose(x.cpu().double(), want_x, atol=1e-5)
