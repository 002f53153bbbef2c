"""The Fomatar decoder on the device against the plain implementation (tests/plain_fomatar.py):
whole prompts, decoding through cache and state, portions down to two tokens, unequal batches
against each sequence alone, slots and pages used again, long decoding, greedy generation through
the library's entry point, and the kernels of each mechanism alone with inputs made so that a
window's edge, a far key or a first token shows."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_fomatar as pf
from fomatar_models import CONFIGS, as_float64, write_model
import helpers
from helpers import assert_same_engine, tokens

pytestmark = pytest.mark.gpu

SEEDS = {"mixed": 11, "plain": 12, "from_start": 13, "wide": 14, "delta_only": 15}
LENGTHS = {"mixed": 41, "plain": 150, "from_start": 23, "wide": 140, "delta_only": 70}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, cfg in CONFIGS.items():
        d = str(tmp_path_factory.mktemp("fomatar_" + name))
        out[name] = (d, as_float64(write_model(d, cfg, SEEDS[name], ranks=(8, 16) if name != "plain" else (5, 11))))
    return out


def assert_close(got, ref, dtype, what=""):
    """float32: the library's tolerances. bfloat16: a state carried over hundreds of tokens and a stretch of layers
    run several times pass a rounding error on, so single rows may be off by more than a dense decoder's 3e-2 of
    the largest logit; the mean error, which a fault in a mechanism moves first, keeps a tight bound."""
    if dtype == "float32":
        return helpers.assert_close(got, ref, dtype, what)
    worst = float(helpers.row_errors(got, ref).max())
    assert worst <= 8e-2, f"{what}: a row is off by {worst:.3e} of its largest logit (bfloat16)"
    mean = helpers.mean_err(got, ref)
    assert mean <= 6e-3, f"{what}: mean error {mean:.3e} (bfloat16)"


_models: dict = {}


def model(folders, name, dtype):
    import camelid_b200
    if (name, dtype) not in _models:
        _models[(name, dtype)] = camelid_b200.load(folders[name][0], dtype=dtype)
    return _models[(name, dtype)]


_plain: dict = {}


def plain(folders, name, ids):
    key = (name, tuple(ids))
    if key not in _plain:
        _plain[key] = pf.forward(list(ids), folders[name][1], CONFIGS[name])
    return _plain[key]


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
    decoded = run_cut(lm, cache, ids, [n - min(n - 1, 24)])            # the last tokens one by one (captured steps)
    assert_close(decoded, ref, dtype, f"{name} decoded")
    if dtype == "float32":
        assert_same_engine(whole, decoded, f"{name} whole against decoded", tol=1e-5)
    lm.model.check_device_errors()
    cache.book.audit()


@pytest.mark.parametrize("name,cut", [("mixed", [7, 2, 3, 2, 13, 1, 1, 2]), ("plain", [64, 2, 63, 1, 2, 5]),
                                      ("from_start", [1, 2, 2, 3]), ("wide", [2, 126, 2, 3])])
def test_portions_of_a_prompt(cuda, folders, name, cut):
    lm = model(folders, name, "float32")
    ids = tokens(SEEDS[name], LENGTHS[name], CONFIGS[name]["vocab"])
    cache = lm.new_cache(1024)
    got = run_cut(lm, cache, ids, cut)
    assert_close(got, plain(folders, name, ids), "float32", f"{name} in portions {cut}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "plain", "wide"])
def test_unequal_batch_against_each_alone(cuda, folders, name, dtype):
    """Prompts of 1, 17 and 90 tokens start together, are decoded together and end one after the other."""
    from camelid_b200.engine.model import StepEntry
    lm = model(folders, name, dtype)
    vocab = CONFIGS[name]["vocab"]
    seqs = [tokens(100 + i, n, vocab) for i, n in enumerate((9, 30, 110))]
    prompt = [1, 17, 90]
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
    """A cache of three pages: every sequence gets the slot and the pages the one before gave back."""
    lm = model(folders, "plain", "float32")
    cache = lm.new_cache(192, max_slots=1)
    for i, n in enumerate((130, 75, 140)):
        ids = tokens(200 + i, n, CONFIGS["plain"]["vocab"])
        got = run_cut(lm, cache, ids, [n - 10])
        assert_close(got, plain(folders, "plain", ids), "float32", f"sequence {i} in a slot used before")
        cache.book.audit()
    assert cache.book.slots.n_free == 1 and all(p.n_free == p.n for p in cache.book.pools)


def test_long_decoding(cuda, folders):
    lm = model(folders, "mixed", "float32")
    ids = tokens(5, 260, CONFIGS["mixed"]["vocab"])
    cache = lm.new_cache(512)
    got = run_cut(lm, cache, ids, [3])
    assert_close(got, plain(folders, "mixed", ids), "float32", "257 tokens decoded one by one")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(cuda, folders, dtype):
    """``generate`` (scheduler, batches, the decode loop on the device) picks the plain implementation's tokens."""
    lm = model(folders, "mixed", dtype)
    P, cfg = folders["mixed"][1], CONFIGS["mixed"]
    prompts = [tokens(300, 5, cfg["vocab"]), tokens(301, 19, cfg["vocab"]), tokens(302, 1, cfg["vocab"])]
    for _ in range(2):                                         # the second call uses the slots again
        out = lm.generate(prompts, max_tokens=9)
        for p, new in zip(prompts, out):
            assert len(new) == 9
            seq = list(p)
            for tok in new:
                ref = pf.forward(seq, P, cfg)[-1]
                top2 = torch.topk(ref, 2).values
                if dtype == "float32" or float(top2[0] - top2[1]) > 0.25:      # bfloat16 may flip a near tie
                    assert tok == int(ref.argmax()), (seq, new)
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


def test_trace_runner_replays_a_fomatar_model(cuda, folders, tmp_path):
    folder, P = folders["from_start"]
    cfg = CONFIGS["from_start"]
    a, b = tokens(1, 9, cfg["vocab"]), tokens(2, 4, cfg["vocab"])
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:7], "want": [0, 6]}, {"id": "b", "tokens": b[:1], "want": [0]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[7:8], "want": []}, {"id": "b", "tokens": b[1:2], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[8:9], "want": [0]}, {"id": "b", "tokens": b[2:3], "want": [0]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": b[3:4], "want": [0]}], "end": ["b"]}]
    exe = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "trace_run")
    r = subprocess.run([sys.executable, exe, "--model", folder, "--dtype", "float32", "--out", str(tmp_path), "--max-tokens", "128"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == [f"done {i}" for i in range(4)]
    ra, rb = pf.forward(a, P, cfg), pf.forward(b, P, cfg)
    want = {0: torch.stack([ra[0], ra[6], rb[0]]), 1: rb[1:2], 2: torch.stack([ra[8], rb[2]]), 3: rb[3:4]}
    for i, ref in want.items():
        got = torch.from_numpy(np.fromfile(tmp_path / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"]))
        assert_close(got, ref, "float32", f"step {i}")


# ---- each mechanism's kernels alone -------------------------------------------------------------

def arrays(cuda, starts, news):
    """The packed-row arrays of a step: one slot per sequence, slot = its index."""
    row_seq = np.repeat(np.arange(len(news)), news)
    row0 = np.concatenate([[0], np.cumsum(news)[:-1]])
    row_pos = np.concatenate([np.arange(s, s + n) for s, n in zip(starts, news)])
    dev = lambda a: torch.as_tensor(np.asarray(a), dtype=torch.int32, device=cuda)      # noqa: E731
    return {"row_seq": dev(row_seq), "row_pos": dev(row_pos), "seq_row0": dev(row0), "seq_new": dev(news),
            "seq_start": dev(starts), "seq_slot": dev(np.arange(len(news)))}


def portions(n, cut):
    sizes = list(cut) + [1] * (n - sum(cut))
    at = 0
    for s in sizes:
        yield at, s
        at += s


@pytest.mark.parametrize("cut", [[200], [64, 2, 70], [1]])
def test_bigram_embedding_and_token_shift_kernels(cuda, cut):
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(0)
    V, W, B = 50, 24, 13
    table, bigram = torch.randn(V, W, generator=gen), torch.randn(B + 1, W, generator=gen)
    mix = torch.rand(W, generator=gen)
    ids = tokens(4, 200, V)
    cfg = {"embedding": {"bigram": {"buckets": B, "mul_prev": 1000003, "mul_cur": 7}}}
    ref = pf.embedding(ids, {"embed": table.double(), "bigram": bigram.double()}, cfg)
    ref_shift = pf.token_shift(ref, mix.double())
    prev = torch.full((3,), 77, dtype=torch.int32, device=cuda)          # stale state of an earlier user of the slot
    state = torch.full((3, 1, W), 9.0, device=cuda)
    err = torch.zeros(1, dtype=torch.int32, device=cuda)
    got, got_shift = [], []
    for at, n in portions(200, cut):
        a = arrays(cuda, [at], [n])
        out = torch.empty(n, W, device=cuda)
        ops.bigram_embed(table.to(cuda), bigram.to(cuda), torch.tensor(ids[at:at + n], dtype=torch.int32, device=cuda), a["row_seq"],
                         a["row_pos"], a["seq_row0"], a["seq_new"], a["seq_slot"], prev, out, 1, B, 1000003, 7, err)
        shifted = torch.empty_like(out)
        ops.token_shift(out, mix.to(cuda), state, a["row_seq"], a["row_pos"], a["seq_row0"], a["seq_slot"], shifted)
        ops.keep_last_rows(out, 0, W, state, a["seq_row0"], a["seq_new"], a["seq_start"], a["seq_slot"], 1)
        got.append(out.cpu())
        got_shift.append(shifted.cpu())
    assert torch.allclose(torch.cat(got).double(), ref, atol=1e-6)
    assert torch.allclose(torch.cat(got_shift).double(), ref_shift, atol=1e-6)
    assert int(err.item()) == 0 and int(prev[0]) == ids[-1] and int(prev[1]) == 77


def _paged(cuda, T, G, D, Dv, dtype):
    pages = (T + 63) // 64
    order = list(range(pages))[::-1]                                   # pages in another order than positions
    table = torch.tensor([order + [-1]], dtype=torch.int32, device=cuda)
    k = torch.full((pages + 1, G, 64, D), float("nan"), dtype=dtype, device=cuda)
    v = torch.full((pages + 1, G, 64, Dv), float("nan"), dtype=dtype, device=cuda)
    return table, k, v


@pytest.mark.parametrize("cut", [[210], [100, 2, 60], [5]])
def test_window_attention_kernels_at_the_windows_edge(cuda, cut):
    """One key a query loves stands just inside the window for some rows and just outside for the next: the output
    jumps from that key's value to the others' mean. Window 70 over pages of 64, keys and values of different sizes."""
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(1)
    T, H, G, D, Dv, window, scale = 210, 4, 2, 24, 40, 70, 0.2
    q = torch.randn(T, H, D, generator=gen) * 0.3
    k = torch.randn(T, G, D, generator=gen) * 0.3
    v = torch.randn(T, G, Dv, generator=gen)
    for j in (0, 63, 64, 100):                                         # loved keys: a first token, a page's edges
        k[j] = 0.0
        k[j, :, 0] = 40.0
    q[:, :, 0] = 3.0
    r1, r2 = torch.tensor([0.0, 1.0, 2.0, 0.5]), torch.tensor([0.3, 0.2, 0.05, 0.4])
    gate = torch.randn(T, H * Dv, generator=gen)
    qw, kw = 1.0 + 0.3 * torch.randn(D, generator=gen), 1.0 + 0.3 * torch.randn(D, generator=gen)
    eps = 1e-5
    ref = pf.window_scores_core(pf.rms_norm(q.double(), qw.double(), eps), pf.rms_norm(k.double(), kw.double(), eps), v.double(),
                                scale, window, r1.double(), r2.double()).reshape(T, H * Dv) * torch.sigmoid(gate.double())
    # rows whose loved key has just left the window differ from those that still see it
    assert float((ref[169] - ref[170]).abs().max()) > 0.1
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1), gate], 1).to(cuda)
    table, kp, vp = _paged(cuda, T, G, D, Dv, torch.float32)
    got = []
    for at, n in portions(T, cut):
        a = arrays(cuda, [at], [n])
        qn = torch.empty(n, H * D, device=cuda)
        ops.qk_norm_kv_write(proj[at:at + n], qw.to(cuda), kw.to(cuda), eps, a["row_seq"], a["row_pos"], table, qn, kp, vp, H, G, D, Dv)
        out = torch.empty(n, H * Dv, device=cuda)
        ops.window_attention(qn, kp, vp, table, a["row_seq"], a["row_pos"], r1.to(cuda), r2.to(cuda), proj[at:at + n],
                             H * D + G * D + G * Dv, out, H, G, D, Dv, window, scale)
        got.append(out.cpu())
    got = torch.cat(got).double()
    assert torch.isfinite(got).all()
    assert float((got - ref).abs().max()) < 2e-5 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("D,group,window", [(64, 3, 70), (128, 2, 200), (128, 1, 33)])
def test_prompt_attention_on_tensor_cores_against_the_plain_formula(cuda, D, group, window):
    """bfloat16 prompts with keys and values of 64 or 128 channels take the tcgen05 kernel with the distance penalty in
    its softmax: against the plain formula on the same bfloat16 q, k, v (two sequences, the second from position 0 too)."""
    from camelid_b200.csrc import ops
    from camelid_b200.parts import linear
    gen = torch.Generator().manual_seed(7)
    G, lens = 2, [230, 67]
    H = G * group
    r1, r2 = torch.rand(H, generator=gen) * 2.5, torch.rand(H, generator=gen) * 0.5
    scale = D ** -0.5
    rows, tiles_hpc_chunks = sum(lens), ops.attn_tc_tiling(H, G)
    tile_rows, hpc, chunks = tiles_hpc_chunks
    q = (torch.randn(rows, H, D, generator=gen)).to(torch.bfloat16)
    k = (torch.randn(rows, G, D, generator=gen)).to(torch.bfloat16)
    v = (torch.randn(rows, G, D, generator=gen)).to(torch.bfloat16)
    ref, at = [], 0
    for n in lens:
        ref.append(pf.window_scores_core(q[at:at + n].double(), k[at:at + n].double(), v[at:at + n].double(), scale, window,
                                         r1.double(), r2.double()).reshape(n, H * D))
        at += n
    ref = torch.cat(ref)
    pages = [(n + 63) // 64 for n in lens]
    width = max(pages)
    table = torch.full((2, width), -1, dtype=torch.int32)
    table[0, :pages[0]] = torch.arange(pages[0]) + pages[1]
    table[1, :pages[1]] = torch.arange(pages[1])
    table = table.to(cuda)
    kp = torch.zeros(sum(pages), G, 64, D, dtype=torch.bfloat16, device=cuda)
    vp = torch.zeros_like(kp)
    a = arrays(cuda, [0, 0], lens)
    proj = torch.cat([q.reshape(rows, -1), k.reshape(rows, -1), v.reshape(rows, -1)], 1).float().to(cuda)
    qn = torch.empty(rows, H * D, dtype=torch.bfloat16, device=cuda)
    ops.qk_norm_kv_write(proj, None, None, 1e-6, a["row_seq"], a["row_pos"], table, qn, kp, vp, H, G, D, D)
    tile_seq = [s for s, n in enumerate(lens) for _ in range(0, n, tile_rows)]
    tile_q0 = [q0 for n in lens for q0 in range(0, n, tile_rows)]
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device=cuda)      # noqa: E731
    out = torch.empty(rows, H * D, dtype=torch.bfloat16, device=cuda)
    assert ops.attn_tc_usable(qn, out, D)
    ops.attn_prefill_tc(qn, out, kp, vp, table, dev(tile_seq), dev(tile_q0), len(tile_seq), a["seq_row0"], a["seq_start"],
                        a["seq_new"], H, G, D, tile_rows, hpc, chunks, window, scale, linear._err_word(cuda), r1.to(cuda), r2.to(cuda))
    plain_kernel = torch.empty_like(out)
    ops.window_attention(qn, kp, vp, table, a["row_seq"], a["row_pos"], r1.to(cuda), r2.to(cuda), None, 0, plain_kernel, H, G, D, D,
                         window, scale)
    linear.check_errors()
    for got, what in ((out, "tensor cores"), (plain_kernel, "plain kernel")):
        err = float((got.cpu().double() - ref).abs().max())
        assert err < 3e-2, f"{what}: {err}"


@pytest.mark.parametrize("cut", [[300], [3, 2, 200], [1]])
def test_scan_kernels_keep_a_far_key(cuda, cut):
    """A key written at token 2 and asked for at token 290, with decays close to one: the state carries it through
    prompts, portions and single steps. Both scans, with heads whose value size is no multiple of the block."""
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(2)
    T, H, G, D, Dv = 300, 4, 2, 20, 37
    # ---- delta rule
    q = pf.unit(torch.randn(T, G, D, generator=gen).double()) * D ** -0.5
    k = pf.unit(torch.randn(T, G, D, generator=gen).double())
    k[2] = 0.0
    k[2, :, 5] = 1.0
    k[3:, :, 5] = 0.0                                   # nobody overwrites that channel
    q[290] = 0.0
    q[290, :, 5] = 1.0
    v = torch.randn(T, H, Dv, generator=gen).double()
    beta_in = torch.randn(T, H, generator=gen)
    decay_in = torch.randn(T, H * D, generator=gen) - 6.0
    a_log, dt_bias = torch.randn(H, generator=gen) - 2.0, torch.randn(H * D, generator=gen) * 0.1
    decay = torch.exp(-torch.exp(a_log.double()).view(1, H, 1) * pf.softplus(decay_in.double() + dt_bias.double()).view(T, H, D))
    ref = pf.delta_core(q, k, v, torch.sigmoid(beta_in.double()), decay).reshape(T, H * Dv)
    assert float(ref[290].abs().max()) > 0.05
    qkv = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1).float().to(cuda)
    state = torch.full((2, H, Dv, D), 5.0, device=cuda)                # stale: a sequence that starts here reads none of it
    got = []
    for at, n in portions(T, cut):
        a = arrays(cuda, [at], [n])
        out = torch.empty(n, H * Dv, device=cuda)
        ops.delta_scan(qkv[at:at + n], beta_in[at:at + n].to(cuda), 0, decay_in[at:at + n].to(cuda), a_log.to(cuda), dt_bias.to(cuda),
                       state, a["seq_row0"], a["seq_new"], a["seq_start"], a["seq_slot"], out, 1, H, G, D, Dv)
        got.append(out.cpu())
    got = torch.cat(got).double()
    assert float((got - ref).abs().max()) < 1e-4 * float(ref.abs().max())
    assert float(state[1].min()) == 5.0
    # ---- matrix memory: q, k, v, gates as columns of one projection
    q = torch.randn(T, H, D, generator=gen)
    k = torch.randn(T, H, D, generator=gen)
    v = torch.randn(T, H, Dv, generator=gen)
    gi_in, gf_in = torch.randn(T, H, generator=gen) * 3.0, torch.randn(T, H, generator=gen) * 3.0
    bi, bf, cap = torch.randn(H, generator=gen), torch.randn(H, generator=gen) + 4.0, 6.0
    gi = cap * torch.tanh((gi_in.double() + bi.double()) / cap)
    gf = pf.logsigmoid(cap * torch.tanh((gf_in.double() + bf.double()) / cap))
    ref = pf.matrix_memory_core(q.double() * D ** -0.5, k.double(), v.double(), gi, gf)
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1), gi_in, gf_in], 1).to(cuda)
    cols = (0, H * D, 2 * H * D, 2 * H * D + H * Dv, 2 * H * D + H * Dv + H)
    state = torch.full((2, H, Dv + 1, D), 5.0, device=cuda)
    state_m = torch.full((2, H, Dv + 1), 5.0, device=cuda)
    got = []
    for at, n in portions(T, cut):
        a = arrays(cuda, [at], [n])
        raw = torch.empty(n, H, Dv + 2, device=cuda)
        ops.memory_scan(proj[at:at + n], cols, bi.to(cuda), bf.to(cuda), cap, D ** -0.5, state, state_m, a["seq_row0"], a["seq_new"],
                        a["seq_start"], a["seq_slot"], raw, 1, H, D, Dv)
        got.append(raw.cpu())
    raw = torch.cat(got).double()
    den = torch.maximum(raw[..., Dv].abs(), torch.exp(-raw[..., Dv + 1])) + 1e-6
    got = raw[..., :Dv] / den.unsqueeze(-1)
    assert float((got - ref).abs().max()) < 1e-4 * float(ref.abs().max())


def test_convolution_and_unit_norm_kernel_over_portions(cuda):
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(3)
    T, H, G, D, Dv, taps = 40, 3, 1, 12, 20, 4
    C = 2 * G * D + H * Dv
    x = torch.randn(T, C + 5, generator=gen)                       # further columns behind the channels
    w = torch.randn(C, taps, generator=gen)
    y = pf.silu(pf.short_conv(x[:, :C].double(), w.double()))
    ref = torch.cat([(pf.unit(y[:, :G * D].view(T, G, D)) * D ** -0.5).reshape(T, -1),
                     pf.unit(y[:, G * D:2 * G * D].view(T, G, D)).reshape(T, -1), y[:, 2 * G * D:]], 1)
    state = torch.full((1, taps - 1, C), 3.0, device=cuda)
    got = []
    for at, n in portions(T, [2, 1, 7, 2]):
        a = arrays(cuda, [at], [n])
        out = torch.empty(n, C, device=cuda)
        src = x[at:at + n].to(cuda)
        ops.conv_unit(src, w.to(cuda), state, a["row_seq"], a["row_pos"], a["seq_row0"], a["seq_slot"], out, G, H, D, Dv, D ** -0.5)
        ops.keep_last_rows(src, 0, C, state, a["seq_row0"], a["seq_new"], a["seq_start"], a["seq_slot"], 1)
        got.append(out.cpu())
    assert float((torch.cat(got).double() - ref).abs().max()) < 1e-5


def test_read_out_norm_combine_gelu_and_cap_kernels(cuda):
    from camelid_b200.csrc import ops
    gen = torch.Generator().manual_seed(4)
    rows, H, Dv, W = 9, 3, 37, 50
    raw = torch.randn(rows, H, Dv, generator=gen)
    w = 1.0 + 0.2 * torch.randn(Dv, generator=gen)
    gate = torch.randn(rows, H * Dv + 3, generator=gen)
    out = torch.empty(rows, H * Dv, device=cuda)
    ops.head_norm_gate(raw.to(cuda), False, w.to(cuda), False, gate.to(cuda), 3, out, H, Dv, 1e-5)
    ref = (pf.rms_norm(raw.double(), w.double(), 1e-5).reshape(rows, -1) * torch.sigmoid(gate[:, 3:].double()))
    assert float((out.cpu().double() - ref).abs().max()) < 1e-5
    # the mean of two normed branches, one of them in split sums
    a, b = torch.randn(rows, W, generator=gen), torch.randn(3, rows, W, generator=gen)
    wa, wb = torch.randn(W, generator=gen), torch.randn(W, generator=gen)
    res = torch.randn(rows, W, generator=gen)
    got = res.clone().to(cuda)
    ops.norm_combine([(a.to(cuda), wa.to(cuda)), (b.to(cuda), wb.to(cuda))], got, 1e-5, 0.5)
    ref = res.double() + 0.5 * (pf.rms_norm(a.double(), wa.double(), 1e-5) + pf.rms_norm(b.double().sum(0), wb.double(), 1e-5))
    assert float((got.cpu().double() - ref).abs().max()) < 1e-5
    x = torch.randn(1000, generator=gen) * 3
    g = x.clone().to(cuda)
    ops.gelu_tanh_(g)
    assert float((g.cpu().double() - pf.gelu_tanh(x.double())).abs().max()) < 1e-6
    c = (x * 10).to(cuda)
    ops.softcap_(c, 7.0)
    assert float((c.cpu().double() - 7.0 * torch.tanh(x.double() * 10 / 7.0)).abs().max()) < 1e-5
