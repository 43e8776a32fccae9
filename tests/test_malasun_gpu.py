"""The layered engine on a B200 against the plain Malasun restatement (oracle/malasun.py): every mechanism alone, prompts cut into
portions, decoding through the cache and the state slots, mixed batches, pages and slots that are used again, window edges and far
keys made visible by a token whose embedding is scaled up, other sizes, and greedy generation through the library's own entries."""
import numpy as np
import pytest

from aha_b200 import synth
from conftest import has_gpu

pytestmark = pytest.mark.gpu
if not has_gpu():
    pytest.skip("needs a GPU", allow_module_level=True)

from aha_b200 import B200Model          # noqa: E402
from oracle.malasun import Malasun      # noqa: E402

TOL32 = 2e-4     # exact mode: fp32 everywhere against float64
TOL16 = 6e-2     # serving mode: bf16 products


def A(heads=2, kv_heads=1, dim=16, vdim=16, window=None, conv=None, kv_from=None, ff=None, scale=None):
    d = {"type": "attention", "heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "window": window, "conv": conv, "kv_from": kv_from, "ff": ff}
    if scale is not None:
        d["scale"] = scale
    return d


def R(heads=2, dim=8, vdim=8, ff=None):
    return {"type": "hgrn2", "heads": heads, "dim": dim, "vdim": vdim, "ff": ff}


class Pair:
    """The library's handle and the oracle on the same random checkpoint."""

    def __init__(self, cfg, seed=0, exact=True, max_ctx=1024, max_seqs=4, step_tokens=512, boost=None, plain=False, edit=None):
        self.cfg = cfg
        w = synth.make_malasun(cfg, seed)
        f = {k: synth.bf16_to_f32(v) for k, v in w.items()}
        if boost is not None:       # one token's embedding scaled up (still bf16-exact): its key / value stand out wherever it is visible
            f["embed"] = f["embed"].copy()
            f["embed"][boost] *= 8.0
            w["embed"] = synth._bf16_round(f["embed"])
        if edit is not None:        # edit(name, values) -> new values or None, for every tensor
            for k in list(f):
                a = edit(k, f[k])
                if a is not None:
                    w[k] = synth._bf16_round(np.asarray(a, np.float32))
                    f[k] = synth.bf16_to_f32(w[k])
        self.m = B200Model("malasun", cfg, w, max_ctx=max_ctx, max_prefill=step_tokens, max_seqs=max_seqs, exact_fp32=exact, attn_impl=1 if plain else 0)
        self.o = Malasun(cfg, f)
        self.tol = TOL32 if exact else TOL16
        self.V = cfg["vocab"]

    def ids(self, n, seed=0, avoid=None):
        r = np.random.default_rng(seed).integers(0, self.V, n)
        if avoid is not None:
            r[r == avoid] = (avoid + 1) % self.V
        return r.astype(np.uint32)

    def check(self, got, want, what=""):
        want = np.asarray(want, np.float64)
        err = np.abs(got - want).max() / max(1.0, want.std())
        assert err <= self.tol, f"{what}: logits differ from the plain implementation by {err:.3e}"

    def run_cuts(self, ids, cuts):
        """One sequence fed in portions ending at `cuts`; all logits."""
        s = self.m.seq_open()
        out, a = [], 0
        for b in list(cuts) + [len(ids)]:
            if b > a:
                out.append(self.m.feed([(s, ids[a:b], range(b - a))]))
                a = b
        self.m.seq_close(s)
        return np.concatenate(out)

    def close(self):
        self.m.close()


MECHANISMS = {
    "hgrn2": [R(heads=3, dim=8, vdim=24)],
    "hgrn2_ff": [R(heads=1, dim=16, vdim=8, ff=40)],
    "attn_plain": [A(heads=4, kv_heads=2, dim=8, vdim=16)],
    "attn_window": [A(heads=2, kv_heads=2, dim=16, vdim=8, window=7)],
    "attn_window_1": [A(heads=2, kv_heads=1, dim=8, vdim=8, window=1, conv=2)],
    "attn_conv": [A(heads=3, kv_heads=1, dim=8, vdim=8, conv=5, ff=24)],
    "attn_shared": [A(heads=4, kv_heads=2, dim=8, vdim=8, window=33, conv=3), A(heads=4, kv_heads=2, dim=8, vdim=8, window=9, conv=4, kv_from=0)],
    "attn_scale": [A(heads=6, kv_heads=3, dim=12, vdim=20, window=20, scale=0.7)],
}


@pytest.mark.parametrize("name", sorted(MECHANISMS))
def test_each_mechanism_alone(name):
    p = Pair(synth.malasun_config(MECHANISMS[name], width=40, vocab=77), seed=5)
    ids = p.ids(45, 1)
    trace = []
    want = p.o.forward(ids, None, trace)
    p.m.set_trace(True)
    s = p.m.seq_open()
    got = p.m.feed([(s, ids, range(len(ids)))])
    p.check(got, want, name)
    for l, x in enumerate(trace):       # the residual stream after every layer
        h = p.m.debug_read("hidden", l, x.size).reshape(x.shape)
        assert np.abs(h - x).max() <= TOL32 * max(1.0, np.abs(x).max()), f"{name}: layer {l}"
    p.m.seq_close(s)
    # the same tokens one by one, and in portions
    p.check(p.run_cuts(ids, range(1, len(ids))), want, name + " token by token")
    p.check(p.run_cuts(ids, [2, 4, 9, 10, 31, 33]), want, name + " in portions")
    p.close()


@pytest.mark.parametrize("exact", [True, False])
def test_whole_model_portions_and_decoding(exact):
    p = Pair(synth.get_config("malasun", "tiny"), seed=2, exact=exact)
    ids = p.ids(150, 3)
    want = p.o.forward(ids)
    p.check(p.run_cuts(ids, []), want, "whole")
    p.check(p.run_cuts(ids, [2, 4, 5, 8, 15, 31, 32, 33, 64, 96, 97, 127, 129]), want, "portions of 1, 2, 3, 7 and more tokens, at page and window borders")
    p.check(p.run_cuts(ids, list(range(60, 150))), want, "prompt then 90 decoded tokens (past every window)")
    p.check(p.run_cuts(ids, list(range(1, 12))), want, "the first tokens one by one")
    p.close()


def test_tensor_core_linears_in_serving_mode():
    # sizes that tile (K % 64 == 0, N % 32 == 0): portions of 32 tokens and more run their Linear layers on the tcgen05 kernels with
    # bf16 operands, shorter ones and decode steps on the CUDA cores; both must agree with the plain implementation
    cfg = synth.malasun_config([A(heads=4, kv_heads=2, dim=32, vdim=32, window=48, conv=4, ff=256), R(heads=2, dim=32, vdim=64, ff=None),
                                A(heads=4, kv_heads=2, dim=32, vdim=32, window=20, conv=2, kv_from=0, ff=128)], width=128, vocab=160)
    p = Pair(cfg, seed=21, exact=False, max_ctx=2048, step_tokens=2048)
    ids = p.ids(1300, 4)
    want = p.o.forward(ids)
    got = p.run_cuts(ids, [])                       # one 1300-row launch: the CTA-pair kernel for N >= 256, 128 x 128 tiles below
    err = np.abs(got - want).max() / want.std()
    assert err < 2e-3, err                          # bf16 hi + lo operands: far inside the bf16 budget
    p.check(p.run_cuts(ids[:300], [40, 45, 200, 260] + list(range(261, 300))), want[:300], "tensor-core portions beside CUDA-core ones")
    st = p.m.stats()
    assert st["kernel_launches"] > 0
    p.close()


def test_tensor_core_attention_in_serving_mode():
    # head sizes 64 and 128 with dim == vdim: prompt portions of 32 tokens and more run their attention on the tcgen05 flash kernel (window,
    # distance penalty and gate inside it), shorter portions and decoded tokens on the CUDA-core kernel; the marked token's key and value
    # stand out, so a window that is one key off, or a tile that is skipped wrongly, moves the rows around the edges far beyond the budget
    mark = 3
    cfg = synth.malasun_config([A(heads=4, kv_heads=2, dim=64, vdim=64, window=100, conv=4, ff=128), R(heads=2, dim=32, vdim=16),
                                A(heads=4, kv_heads=2, dim=64, vdim=64, window=37, conv=2, kv_from=0), A(heads=2, kv_heads=1, dim=128, vdim=128, window=None, conv=None, ff=64),
                                A(heads=2, kv_heads=2, dim=128, vdim=128, window=130, conv=3)], width=64, vocab=90)
    p = Pair(cfg, seed=31, exact=False, max_ctx=2048, step_tokens=1024, boost=mark)
    ids = p.ids(700, 6, avoid=mark)
    ids[[5, 200, 263, 455]] = mark
    want = p.o.forward(ids)
    for cuts in ([], [40, 45, 300, 333, 429, 461, 600], [130, 131, 194, 195, 259] + list(range(640, 700))):
        got = p.run_cuts(ids, cuts)
        err = np.abs(got - want).max() / want.std()
        assert err < 3e-3, (cuts[:4], err, int(np.abs(got - want).max(axis=1).argmax()))
    # the rows just past every window edge of a marked key depend on the edge being exact
    other = Malasun(synth.malasun_config([A(heads=4, kv_heads=2, dim=64, vdim=64, window=101, conv=4, ff=128), R(heads=2, dim=32, vdim=16),
                                          A(heads=4, kv_heads=2, dim=64, vdim=64, window=38, conv=2, kv_from=0), A(heads=2, kv_heads=1, dim=128, vdim=128, window=None, conv=None, ff=64),
                                          A(heads=2, kv_heads=2, dim=128, vdim=128, window=131, conv=3)], width=64, vocab=90), p.o.w).forward(ids)
    assert np.abs(other[300] - want[300]).max() / want.std() > 0.03        # ten times the budget above
    p.close()


def test_plain_kernels_agree_with_the_fast_ones():
    cfg = synth.get_config("malasun", "tiny")
    ids = np.random.default_rng(3).integers(0, cfg["vocab"], 300).astype(np.uint32)
    out = []
    for plain in (False, True):
        p = Pair(cfg, seed=17, plain=plain)
        out.append(p.run_cuts(ids, [70, 71, 200] + list(range(250, 300))))
        p.check(out[-1], p.o.forward(ids), "plain kernels" if plain else "fast kernels")
        p.close()
    assert np.abs(out[0] - out[1]).max() <= 2 * TOL32 * max(1.0, np.abs(out[1]).std())


def test_recurrence_sizes_beyond_one_column_slice():
    # vdim that is no multiple of the 16-column slice, dim that is no multiple of 4 (unaligned rows), dim above 128 (several state rows per thread)
    for layers in ([R(heads=2, dim=6, vdim=21)], [R(heads=1, dim=136, vdim=40, ff=24)], [R(heads=3, dim=20, vdim=16), R(heads=1, dim=260, vdim=8)]):
        p = Pair(synth.malasun_config(layers, width=36, vocab=50), seed=19)
        ids = p.ids(75, 2)
        want = p.o.forward(ids)
        p.check(p.run_cuts(ids, [33, 34, 66] + list(range(67, 75))), want, "recurrence sizes")
        p.close()


def test_long_portions_are_scanned_in_segments():
    # Entries of 256 tokens and more are cut into 64-token segments that are scanned side by side and joined afterwards.  Forget gates
    # held at 63/64 and above keep hundreds of tokens in the state, so a segment that started from the wrong state would show.  Sizes
    # that are no multiples of the kernels' tiles; long entries that start a sequence and that continue one, beside short ones.
    layers = [R(heads=2, dim=72, vdim=40), R(heads=3, dim=8, vdim=8, ff=24), A(heads=2, kv_heads=1, dim=16, vdim=16, window=48, conv=3), R(heads=1, dim=130, vdim=33)]
    slow = lambda k, a: np.full_like(a, 0.984375) if k.endswith("mix.lower") else None
    p = Pair(synth.malasun_config(layers, width=40, vocab=60), seed=23, max_ctx=2048, max_seqs=3, step_tokens=1024, edit=slow)
    reqs = [p.ids(n, 30 + i) for i, n in enumerate([700, 530, 330])]
    want = [p.o.forward(r) for r in reqs]
    slots = [p.m.seq_open() for _ in reqs]
    at, got = [0] * 3, [[] for _ in reqs]
    plan = [[300, 0, 0], [257, 5, 1], [1, 260, 64], [100, 264, 256], [42, 1, 9]]
    for step in plan:
        ent, who = [], []
        for i, n in enumerate(step):
            if n > 0:
                ent.append((slots[i], reqs[i][at[i]:at[i] + n], range(n))); who.append((i, n)); at[i] += n
        lg = p.m.feed(ent)
        r = 0
        for i, n in who:
            got[i].append(lg[r:r + n]); r += n
    for i in range(3):
        assert at[i] == len(reqs[i])
        p.check(np.concatenate(got[i]), want[i], f"request {i} with segmented portions")
    p.close()
    # many heads x columns make the engine choose longer segments (128 tokens for the first prompt, 256 for the second)
    p = Pair(synth.malasun_config([R(heads=8, dim=4, vdim=1184)], width=16, vocab=40), seed=25, max_ctx=2048, max_seqs=2, step_tokens=1100, edit=slow)
    for n, cuts in ((500, [490]), (1060, [30])):
        ids = p.ids(n, n)
        p.check(p.run_cuts(ids, cuts), p.o.forward(ids), f"{n}-token prompt, longer segments")
    p.close()
    # serving mode (bf16 products), one long prompt against its own token-by-token tail
    p = Pair(synth.malasun_config(layers, width=64, vocab=60), seed=24, exact=False, max_ctx=1024, step_tokens=1024, edit=slow)
    ids = p.ids(600, 5)
    p.check(p.run_cuts(ids, [590] + list(range(591, 600))), p.o.forward(ids), "segmented portion in serving mode")
    p.close()


def test_launches_shorter_than_a_step_are_cut_by_the_scheduler():
    p = Pair(synth.get_config("malasun", "tiny"), seed=4, step_tokens=24)      # the engine itself cuts a 100-token entry into 24-token launches
    ids = p.ids(100, 7)
    p.check(p.run_cuts(ids, []), p.o.forward(ids), "launch size 24")
    p.close()


def test_mixed_batches_equal_each_request_alone():
    p = Pair(synth.get_config("malasun", "tiny"), seed=6, max_ctx=1024, max_seqs=4)
    reqs = [p.ids(n, 10 + i) for i, n in enumerate([70, 3, 41, 129])]
    want = [p.o.forward(r) for r in reqs]
    slots = [p.m.seq_open() for _ in reqs]
    at = [0] * len(reqs)
    got = [[] for _ in reqs]
    plan = [[16, 1, 2, 40], [1, 1, 30, 1], [30, 1, 0, 64], [1, 0, 1, 1], [2, 0, 2, 2], [20, 0, 6, 21]]     # portions beside single tokens
    for step in plan:
        ent, who = [], []
        for i, n in enumerate(step):
            n = min(n, len(reqs[i]) - at[i])
            if n > 0:
                ent.append((slots[i], reqs[i][at[i]:at[i] + n], range(n))); who.append((i, n)); at[i] += n
        lg = p.m.feed(ent)
        r = 0
        for i, n in who:
            got[i].append(lg[r:r + n]); r += n
    for i in range(len(reqs)):
        assert at[i] == len(reqs[i])
        p.check(np.concatenate(got[i]), want[i], f"request {i} in a mixed batch")
    p.close()


def test_pages_and_slots_are_used_again():
    p = Pair(synth.get_config("malasun", "tiny"), seed=8, max_ctx=256, max_seqs=2)
    a, b, c, d = p.ids(120, 1), p.ids(100, 2), p.ids(130, 3), p.ids(90, 4)
    sa = p.m.seq_open(); sb = p.m.seq_open()
    with pytest.raises(Exception):
        p.m.seq_open()                                   # both slots are live
    ga = p.m.feed([(sa, a[:100], range(100)), (sb, b[:60], range(60))])
    gb2 = p.m.feed([(sb, b[60:], range(40)), (sa, a[100:], range(20))])
    p.check(np.concatenate([ga[:100], gb2[40:]]), p.o.forward(a), "a")
    p.check(np.concatenate([ga[100:], gb2[:40]]), p.o.forward(b), "b")
    assert p.m.seq_info()["free_tokens"] == 256 - 128 - 128
    with pytest.raises(Exception):
        p.m.feed([(sa, a[:40], [])])                     # the pool is exhausted
    p.m.seq_close(sa)                                    # a's pages and slot go to c while b is still live
    sc = p.m.seq_open()
    assert sc == sa
    gc = p.m.feed([(sc, c[:128], range(128))])
    p.m.seq_close(sb)
    sd = p.m.seq_open()
    g2 = p.m.feed([(sc, c[128:], range(2)), (sd, d, range(90))])
    p.check(np.concatenate([gc, g2[:2]]), p.o.forward(c), "c in a's slot and pages")
    p.check(g2[2:], p.o.forward(d), "d in b's slot and pages")
    p.close()


@pytest.mark.parametrize("decode", [False, True])
def test_window_edges_show(decode):
    win, mark = 24, 5
    cfg = synth.malasun_config([A(heads=2, kv_heads=1, dim=16, vdim=16, window=win, conv=None), R(), A(heads=2, kv_heads=1, dim=16, vdim=16, window=9, conv=2, kv_from=0)], width=32, vocab=50)
    p = Pair(cfg, seed=9, boost=mark)
    ids = p.ids(80, 2, avoid=mark)
    ids[30] = mark                                         # visible to positions 30 .. 30 + win - 1 in layer 0, 30 .. 38 in layer 2
    want = p.o.forward(ids)
    got = p.run_cuts(ids, list(range(28, 80)) if decode else [29, 31, 40])
    p.check(got, want, "window edges")
    # the test has teeth: with the window one token longer the rows just outside the edge move by far more than the tolerance
    cfg2 = synth.malasun_config([A(heads=2, kv_heads=1, dim=16, vdim=16, window=win + 1, conv=None), R(), A(heads=2, kv_heads=1, dim=16, vdim=16, window=10, conv=2, kv_from=0)], width=32, vocab=50)
    other = Malasun(cfg2, p.o.w).forward(ids)
    assert np.abs(other[30 + win] - want[30 + win]).max() > 100 * p.tol and np.abs(other[39] - want[39]).max() > 100 * p.tol
    p.close()


def test_far_key_among_hundreds_and_page_borders():
    mark = 7
    cfg = synth.malasun_config([A(heads=4, kv_heads=2, dim=16, vdim=16, window=None, conv=3, ff=48), R(heads=2, dim=16, vdim=16)], width=48, vocab=60)
    p = Pair(cfg, seed=11, boost=mark, max_ctx=1024, step_tokens=1024)
    ids = p.ids(420, 5, avoid=mark)
    ids[31] = mark                                         # the last token of the first page
    want = p.o.forward(ids)
    plain = ids.copy(); plain[31] = (mark + 2) % 60
    assert np.abs(p.o.forward(plain)[-1] - want[-1]).max() > 50 * p.tol       # the far key matters at the last position
    s = p.m.seq_open()
    g1 = p.m.feed([(s, ids[:380], [31, 32, 63, 64, 379])])
    g2 = [p.m.feed([(s, ids[t:t + 1], [0])]) for t in range(380, 420)]      # decoding across page borders
    p.m.seq_close(s)
    p.check(g1, want[[31, 32, 63, 64, 379]], "prompt rows at page borders")
    p.check(np.concatenate(g2), want[380:], "decoded rows that still see position 31")
    p.close()


def test_long_decoding_keeps_the_recurrent_state():
    cfg = synth.malasun_config([R(heads=2, dim=16, vdim=8), A(heads=2, kv_heads=2, dim=8, vdim=8, window=12, conv=4), R(heads=1, dim=8, vdim=16, ff=32)], width=24, vocab=40)
    p = Pair(cfg, seed=12)
    ids = p.ids(400, 9)
    p.check(p.run_cuts(ids, list(range(3, 400))), p.o.forward(ids), "397 decoded tokens")
    p.close()


def test_greedy_generation_through_the_entry_points():
    cfg = synth.get_config("malasun", "tiny")
    p = Pair(cfg, seed=13, max_seqs=4)
    prompts = [p.ids(n, 20 + i) for i, n in enumerate([9, 40, 1])]
    want = [p.o.greedy(list(pr), 10) for pr in prompts]
    for pr, w in zip(prompts, want):
        toks, usage = p.m.generate(pr, max_tokens=10)
        assert toks == w and usage["completion_tokens"] == 10
    out = p.m.generate_batch([dict(input_ids=pr, max_tokens=10) for pr in prompts])
    assert [o[0] for o in out] == want
    # the batch session: requests join while others decode, a finished one frees its slot
    p.m.batch_open()
    s0, t0, fin = p.m.batch_add(prompts[0], max_tokens=10)
    got = {s0: [t0]}
    for _ in range(3):
        got[s0].append(p.m.batch_step()[s0][0])
    s1, t1, fin = p.m.batch_add(prompts[1], max_tokens=10)
    assert s1 != s0
    got[s1] = [t1]
    live = {s0, s1}
    while live:
        res = p.m.batch_step()
        assert set(res) == live
        for s, (tok, finished) in res.items():
            got[s].append(tok)
            if finished:
                live.discard(s)
    p.m.batch_close()
    assert got[s0] == want[0] and got[s1] == want[1]
    # the single-request trait calls
    lg = p.m.forward_initial(prompts[1], 0)[0, 0]
    p.check(lg[None], p.o.forward(prompts[1])[-1:], "forward_initial")
    p.close()


def test_sampler_runs_on_the_engine():
    cfg = synth.get_config("malasun", "tiny")
    p = Pair(cfg, seed=14)
    pr = p.ids(12, 1)
    a, _ = p.m.generate(pr, max_tokens=8, temperature=0.8, top_p=0.9, top_k=20, seed=5)
    b, _ = p.m.generate(pr, max_tokens=8, temperature=0.8, top_p=0.9, top_k=20, seed=5)
    c, _ = p.m.generate(pr, max_tokens=8, temperature=0.8, top_p=0.9, top_k=20, seed=6)
    assert a == b and len(a) == 8 and all(0 <= t < cfg["vocab"] for t in a + c)
    # against the oracle's sampler on the oracle's logits
    from oracle.sample import Sampler
    samp = Sampler(0.8, 0.9, 20, 1.0, 64, seed=5)
    st = p.o.new_state()
    toks = []
    lg = p.o.forward(pr, st)[-1]
    t = samp.sample_and_push(lg[None, None].astype(np.float32), toks)
    for _ in range(7):
        lg = p.o.forward([t], st)[-1]
        t = samp.sample_and_push(lg[None, None].astype(np.float32), toks)
    assert a == toks
    p.close()
