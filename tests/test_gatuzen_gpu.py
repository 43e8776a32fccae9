"""The layered engine's sandwich template and the Gatuzen mixers on a B200 against the plain restatement (oracle/gatuzen.py): every
mechanism alone, prompts cut into portions, decoding through the caches and the state slots, mixed batches, pages and slots that are
used again, far keys and page borders made visible by a token whose embedding is scaled up, looped layers with a state per pass,
other sizes (also values that a model may happen to make equal or 1), and greedy generation through the library's own entries."""
import numpy as np
import pytest

from aha_b200 import synth
from conftest import has_gpu

pytestmark = pytest.mark.gpu
if not has_gpu():
    pytest.skip("needs a GPU", allow_module_level=True)

from aha_b200 import B200Model          # noqa: E402
from oracle.gatuzen import Gatuzen      # noqa: E402

TOL32 = 2e-4     # exact mode: fp32 everywhere against float64
TOL16 = 6e-2     # serving mode: bf16 products

YARN = {"factor": 3.0, "original": 24, "fast": 4.0, "slow": 0.5}


def G(heads=2, dim=8, vdim=8, tau=8.0, rank=4, moe=None):
    return {"type": "gla", "heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank, "moe": moe}


def M(heads=4, vdim=8, state=8, groups=2, norm_groups=2, conv=4, moe=None):
    return {"type": "mamba2", "heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv, "moe": moe}


def A(heads=3, dim=8, rot_dim=8, vdim=12, kv_rank=16, base=100.0, scaling=YARN, scale=None, moe=None):
    d = {"type": "latent_attention", "heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "base": base, "scaling": scaling, "moe": moe}
    if scale is not None:
        d["scale"] = scale
    return d


def E(experts=5, top=2, ff=24):
    return {"experts": experts, "top": top, "ff": ff}


TINY = dict(layers=[G(heads=2, dim=8, vdim=12, moe=E(6, 2, 20)), M(heads=4, vdim=6, state=8, groups=2, norm_groups=3, conv=3, moe=E(4, 1, 28)),
                    A(heads=3, dim=8, rot_dim=4, vdim=10, kv_rank=12, moe=E(5, 3, 16)), G(heads=1, dim=12, vdim=8, tau=3.0, rank=3)],
            width=48, vocab=83, groups=3, taps=3, residual_mult=0.4, embed_scale=0.7, logit_scale=1.5, loop=(1, 3, 2))


class Pair:
    """The library's handle and the oracle on the same random checkpoint."""

    def __init__(self, cfg, seed=0, exact=True, max_ctx=1024, max_seqs=4, step_tokens=512, boost=None, plain=False, edit=None):
        self.cfg = cfg
        w = synth.make_gatuzen(cfg, seed)
        f = {k: (np.asarray(v) if k.endswith("table") else synth.bf16_to_f32(v)) for k, v in w.items()}
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
        self.m = B200Model("gatuzen", cfg, w, max_ctx=max_ctx, max_prefill=step_tokens, max_seqs=max_seqs, exact_fp32=exact, attn_impl=1 if plain else 0)
        self.o = Gatuzen(cfg, f)
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
        assert err <= self.tol, f"{what}: logits differ from the plain implementation by {err:.3e} (row {int(np.abs(got - want).max(axis=1).argmax())})"

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


def cfg_of(layers, **kw):
    base = dict(width=40, vocab=77, groups=2, taps=3, residual_mult=0.5, embed_scale=1.0, logit_scale=1.0, loop=None)
    base.update(kw)
    return synth.gatuzen_config(layers, **base)


MECHANISMS = {
    "gla": cfg_of([G(heads=3, dim=8, vdim=24)]),
    "gla_one_head_wide": cfg_of([G(heads=1, dim=20, vdim=6, tau=1.0, rank=1)], groups=1),
    "mamba2": cfg_of([M(heads=4, vdim=8, state=16, groups=2, norm_groups=2, conv=4)]),
    "mamba2_one_group": cfg_of([M(heads=3, vdim=12, state=8, groups=1, norm_groups=1, conv=2)], taps=2),
    "mamba2_group_per_head": cfg_of([M(heads=2, vdim=6, state=12, groups=2, norm_groups=4, conv=5)], groups=5, taps=5),
    "latent": cfg_of([A(heads=4, dim=8, rot_dim=8, vdim=16, kv_rank=24)]),
    "latent_plain_rotary": cfg_of([A(heads=2, dim=16, rot_dim=6, vdim=8, kv_rank=10, scaling=None, scale=0.3)], groups=4),
    "latent_one_head": cfg_of([A(heads=1, dim=4, rot_dim=16, vdim=20, kv_rank=8, base=7.0, scaling={"factor": 2.5, "original": 8, "fast": 2.0, "slow": 0.5})]),
    "experts": cfg_of([G(moe=E(7, 2, 20))]),
    "experts_top1": cfg_of([M(moe=E(3, 1, 36))], taps=1),
    "experts_all": cfg_of([A(moe=E(3, 3, 12))], residual_mult=1.0),
    "no_conv_scales": cfg_of([G(moe=E(4, 2, 16)), A()], taps=0, embed_scale=0.25, logit_scale=3.0, groups=8),
    "loop_all": cfg_of([G(moe=E(4, 2, 16)), M()], loop=(0, 2, 3)),
    "loop_tail": cfg_of([A(), G(), M(moe=E(4, 2, 8))], loop=(2, 3, 2)),
    "loop_once": cfg_of([M(), A(moe=E(2, 1, 8)), G()], loop=(0, 1, 1)),
}


@pytest.mark.parametrize("name", sorted(MECHANISMS))
def test_each_mechanism_alone(name):
    p = Pair(MECHANISMS[name], seed=5)
    ids = p.ids(45, 1)
    trace = []
    want = p.o.forward(ids, None, trace)
    p.m.set_trace(True)
    s = p.m.seq_open()
    got = p.m.feed([(s, ids, range(len(ids)))])
    p.check(got, want, name)
    for l, x in enumerate(trace):       # the residual stream after every layer run (a looped layer once per pass)
        h = p.m.debug_read("hidden", l, x.size).reshape(x.shape)
        assert np.abs(h - x).max() <= TOL32 * max(1.0, np.abs(x).max()), f"{name}: run {l}"
    p.m.seq_close(s)
    p.m.set_trace(False)
    # the same tokens one by one, and in portions
    p.check(p.run_cuts(ids, range(1, len(ids))), want, name + " token by token")
    p.check(p.run_cuts(ids, [2, 4, 9, 10, 31, 33]), want, name + " in portions")
    p.close()


@pytest.mark.parametrize("exact", [True, False])
def test_whole_model_portions_and_decoding(exact):
    p = Pair(synth.gatuzen_config(**TINY), seed=2, exact=exact)
    ids = p.ids(150, 3)
    want = p.o.forward(ids)
    p.check(p.run_cuts(ids, []), want, "whole")
    p.check(p.run_cuts(ids, [2, 4, 5, 8, 15, 31, 32, 33, 64, 96, 97, 127, 129]), want, "portions of 1, 2, 3, 7 and more tokens, at page borders")
    p.check(p.run_cuts(ids, list(range(60, 150))), want, "prompt then 90 decoded tokens")
    p.check(p.run_cuts(ids, list(range(1, 12))), want, "the first tokens one by one")
    p.close()


def test_tensor_core_linears_in_serving_mode():
    # sizes that tile (K % 64 == 0, N % 32 == 0, also after padding): portions of 32 tokens and more run their Linear layers on the tcgen05
    # kernels with bf16 operands, shorter ones and decode steps on the CUDA cores; both must agree with the plain implementation
    layers = [G(heads=4, dim=32, vdim=32, rank=8, moe=E(4, 2, 64)), M(heads=4, vdim=32, state=16, groups=2, norm_groups=2, conv=4, moe=E(4, 2, 64)),
              A(heads=4, dim=64, rot_dim=16, vdim=32, kv_rank=64, base=1e4, scaling={"factor": 2.0, "original": 256, "fast": 16.0, "slow": 2.0}, moe=E(3, 1, 128))]
    cfg = cfg_of(layers, width=128, vocab=160, taps=4, residual_mult=0.6, loop=(1, 3, 2))
    p = Pair(cfg, seed=21, exact=False, max_ctx=2048, step_tokens=2048)
    ids = p.ids(700, 4)
    want = p.o.forward(ids)
    got = p.run_cuts(ids, [])
    err = np.abs(got - want).max() / want.std()
    assert err < 3e-3, err                          # bf16 hi + lo operands: far inside the bf16 budget
    p.check(p.run_cuts(ids[:300], [40, 45, 200, 260] + list(range(261, 300))), want[:300], "tensor-core portions beside CUDA-core ones")
    assert p.m.stats()["kernel_launches"] > 0
    p.close()


@pytest.mark.parametrize("dims", [(40, 8, 64), (64, 32, 64), (64, 32, 128), (128, 64, 128)])
def test_tensor_core_latent_attention_in_serving_mode(dims):
    # value sizes 64 and 128 with keys of up to 192 values: prompt portions of 32 tokens and more run on the tcgen05 flash kernel (key rows
    # longer than value rows, zero-padded to a multiple of 64), shorter portions and decoded tokens on the CUDA-core kernels; the marked
    # token's key and value stand out, so a tile that is skipped or masked wrongly moves the rows behind it far beyond the budget
    dim, rot, vdim = dims
    mark = 3
    cfg = cfg_of([A(heads=3, dim=dim, rot_dim=rot, vdim=vdim, kv_rank=64, base=1e4, scaling={"factor": 2.0, "original": 128, "fast": 8.0, "slow": 1.0}, moe=E(3, 2, 64)), G(heads=2, dim=16, vdim=16)],
                 width=64, vocab=90)
    p = Pair(cfg, seed=31, exact=False, max_ctx=2048, step_tokens=1024, boost=mark)
    ids = p.ids(700, 6, avoid=mark)
    ids[[5, 200, 263, 455]] = mark
    want = p.o.forward(ids)
    for cuts in ([], [40, 45, 300, 333, 429, 461, 600], [130, 131, 194, 195, 259] + list(range(640, 700))):
        got = p.run_cuts(ids, cuts)
        err = np.abs(got - want).max() / want.std()
        assert err < 3e-3, (cuts[:4], err, int(np.abs(got - want).max(axis=1).argmax()))
    plain = ids.copy(); plain[455] = (mark + 2) % 90
    assert np.abs(p.o.forward(plain)[461] - want[461]).max() / want.std() > 0.03      # ten times the budget above: the marked key is seen
    p.close()


def test_plain_kernels_agree_with_the_fast_ones():
    cfg = synth.gatuzen_config(**TINY)
    ids = np.random.default_rng(3).integers(0, cfg["vocab"], 300).astype(np.uint32)
    out = []
    for plain in (False, True):
        p = Pair(cfg, seed=17, plain=plain)
        out.append(p.run_cuts(ids, [70, 71, 200] + list(range(250, 300))))
        p.check(out[-1], p.o.forward(ids), "plain kernels" if plain else "fast kernels")
        p.close()
    assert np.abs(out[0] - out[1]).max() <= 2 * TOL32 * max(1.0, np.abs(out[1]).std())


def test_recurrence_sizes_beyond_one_column_slice():
    # vdim that is no multiple of the column slice, dim / state that is no multiple of 4 (unaligned rows) or above 128 and 256
    for layers in ([G(heads=2, dim=6, vdim=21)], [G(heads=1, dim=136, vdim=40, moe=E(3, 2, 8))], [M(heads=3, vdim=21, state=6, groups=3, norm_groups=1)],
                   [M(heads=2, vdim=8, state=132, groups=1), G(heads=1, dim=260, vdim=8)]):
        p = Pair(cfg_of(layers, width=36, vocab=50, groups=3), seed=19)
        ids = p.ids(75, 2)
        want = p.o.forward(ids)
        p.check(p.run_cuts(ids, [33, 34, 66] + list(range(67, 75))), want, "recurrence sizes")
        p.close()


def slow_decay(k, a):
    """Decays close to one keep hundreds of tokens in the state: a segment that started from the wrong state would show."""
    if k.endswith("mix.a2.b"):
        return np.full_like(a, 6.0)
    if k.endswith("mix.a2"):
        return a * 0.1
    if k.endswith("mix.A_log"):
        return np.full_like(a, -4.0)
    return None


def test_long_portions_are_scanned_in_segments():
    # Entries of 256 tokens and more are cut into segments that are scanned side by side and joined afterwards.  Long entries that start a
    # sequence and that continue one, beside short ones; sizes that are no multiples of the kernels' tiles.
    layers = [G(heads=2, dim=72, vdim=40, tau=16.0), M(heads=3, vdim=8, state=24, groups=3, norm_groups=1, moe=E(3, 1, 16)), A(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=8),
              G(heads=1, dim=130, vdim=33, tau=4.0)]
    p = Pair(cfg_of(layers, width=40, vocab=60, loop=(0, 2, 2)), seed=23, max_ctx=2048, max_seqs=3, step_tokens=1024, edit=slow_decay)
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
    # serving mode (bf16 products), one long prompt against its own token-by-token tail
    p = Pair(cfg_of(layers, width=64, vocab=60), seed=24, exact=False, max_ctx=1024, step_tokens=1024, edit=slow_decay)
    ids = p.ids(600, 5)
    p.check(p.run_cuts(ids, [590] + list(range(591, 600))), p.o.forward(ids), "segmented portion in serving mode")
    p.close()


def test_launches_shorter_than_a_step_are_cut_by_the_scheduler():
    p = Pair(synth.gatuzen_config(**TINY), seed=4, step_tokens=24)      # the engine itself cuts a 100-token entry into 24-token launches
    ids = p.ids(100, 7)
    p.check(p.run_cuts(ids, []), p.o.forward(ids), "launch size 24")
    p.close()


def test_mixed_batches_equal_each_request_alone():
    p = Pair(synth.gatuzen_config(**TINY), seed=6, max_ctx=1024, max_seqs=4)
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
    p = Pair(synth.gatuzen_config(**TINY), seed=8, max_ctx=256, max_seqs=2)
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
    p.m.seq_close(sa)                                    # a's pages and slot (states, convolution tails of every run) go to c while b is still live
    sc = p.m.seq_open()
    assert sc == sa
    gc = p.m.feed([(sc, c[:128], range(128))])
    p.m.seq_close(sb)
    sd = p.m.seq_open()
    g2 = p.m.feed([(sc, c[128:], range(2)), (sd, d, range(90))])
    p.check(np.concatenate([gc, g2[:2]]), p.o.forward(c), "c in a's slot and pages")
    p.check(g2[2:], p.o.forward(d), "d in b's slot and pages")
    p.close()


def test_far_key_among_hundreds_and_page_borders():
    mark = 7
    cfg = cfg_of([A(heads=4, dim=16, rot_dim=8, vdim=16, kv_rank=24, moe=E(4, 2, 24)), G(heads=2, dim=16, vdim=16)], width=48, vocab=60)
    p = Pair(cfg, seed=11, boost=mark, max_ctx=1024, step_tokens=1024)
    ids = p.ids(420, 5, avoid=mark)
    ids[31] = mark                                         # the last token of the first page
    want = p.o.forward(ids)
    plain = ids.copy(); plain[31] = (mark + 2) % 60
    assert np.abs(p.o.forward(plain)[-1] - want[-1]).max() > 50 * p.tol       # the far key matters at the last position
    s = p.m.seq_open()
    g1 = p.m.feed([(s, ids[:380], [31, 32, 63, 64, 379])])
    g2 = [p.m.feed([(s, ids[t:t + 1], [0])]) for t in range(380, 420)]      # decoding across page borders, keys split over several blocks
    p.m.seq_close(s)
    p.check(g1, want[[31, 32, 63, 64, 379]], "prompt rows at page borders")
    p.check(np.concatenate(g2), want[380:], "decoded rows that still see position 31")
    p.close()


def test_latent_prompt_portions_of_other_head_sizes():
    # portions of 32 tokens and more expand keys and values and run the tiled kernel (value sizes up to 64, 128 and 256 take different
    # instances; odd sizes leave partial tiles), shorter ones and decoded tokens the absorbed form; both continue one another's cache
    # (18 heads: the decode kernel serves sixteen heads at a time, then the other two)
    for layer in (A(heads=2, dim=20, rot_dim=6, vdim=136, kv_rank=24), A(heads=3, dim=6, rot_dim=2, vdim=5, kv_rank=9), A(heads=1, dim=40, rot_dim=24, vdim=70, kv_rank=32),
                  A(heads=18, dim=8, rot_dim=4, vdim=8, kv_rank=20)):
        p = Pair(cfg_of([layer, G()], width=32, vocab=50), seed=27, max_ctx=1024, max_seqs=3, step_tokens=512)
        ids = p.ids(330, 3)
        want = p.o.forward(ids)
        p.check(p.run_cuts(ids, [70, 75, 140, 141, 205, 269, 300] + list(range(301, 330))), want, "long and short portions in turn")
        a, b = p.ids(200, 4), p.ids(90, 5)
        sa, sb = p.m.seq_open(), p.m.seq_open()
        g1 = p.m.feed([(sa, a[:100], range(100)), (sb, b[:3], range(3))])
        g2 = p.m.feed([(sb, b[3:80], range(77)), (sa, a[100:165], range(65))])          # two long entries, both continuing
        g3 = p.m.feed([(sa, a[165:], range(35)), (sb, b[80:], range(10))])
        p.check(np.concatenate([g1[:100], g2[77:], g3[:35]]), p.o.forward(a), "a")
        p.check(np.concatenate([g1[100:], g2[:77], g3[35:]]), p.o.forward(b), "b")
        p.close()


@pytest.mark.parametrize("seed", range(14))
def test_random_shapes_and_layer_orders(seed):
    # sizes, head counts, layer order, loop span and constants drawn at random (odd sizes included): nothing may rest on one model's values
    r = np.random.default_rng(100 + seed)
    pick = lambda *xs: xs[int(r.integers(0, len(xs)))]
    groups = pick(1, 2, 3, 4)
    width = groups * pick(6, 10, 16, 20)

    def moe():
        n = pick(2, 3, 5, 9)
        return pick(None, E(n, int(r.integers(1, n + 1)), pick(6, 16, 24)))

    def layer():
        t = pick("gla", "mamba2", "latent")
        if t == "gla":
            return G(heads=pick(1, 2, 5), dim=pick(4, 6, 16, 36), vdim=pick(4, 10, 32, 40), tau=pick(1.0, 4.0, 16.0, 64.0), rank=pick(1, 3, 8), moe=moe())
        if t == "mamba2":
            g = pick(1, 2, 3)
            ng = pick(1, 2, 4)
            return M(heads=g * pick(1, 2, 4), vdim=ng * pick(2, 3, 8), state=pick(4, 6, 16, 40), groups=g, norm_groups=ng, conv=pick(1, 2, 4, 7), moe=moe())
        rd = pick(2, 4, 8, 12)
        sc = pick(None, {"factor": pick(2.0, 6.0, 16.0), "original": pick(8, 32, 128), "fast": pick(2.0, 8.0, 32.0), "slow": pick(0.5, 1.0, 2.0)})
        return A(heads=pick(1, 2, 3, 7), dim=pick(4, 6, 16, 24), rot_dim=rd, vdim=pick(4, 6, 16, 36), kv_rank=pick(4, 10, 16, 48), base=pick(10.0, 1e3, 1e6), scaling=sc,
                 scale=pick(None, 0.2, 0.5), moe=moe())

    n = int(r.integers(1, 6))
    layers = [layer() for _ in range(n)]
    a = int(r.integers(0, n + 1)); b = int(r.integers(a, n + 1))
    loop = pick(None, (a, b, pick(1, 2, 3)))
    cfg = synth.gatuzen_config(layers, width=width, vocab=pick(17, 50, 131), eps=pick(1e-6, 1e-5, 1e-3), groups=groups, taps=pick(0, 1, 2, 4, 6),
                               residual_mult=pick(0.2, 0.5, 1.0, 1.7), embed_scale=pick(0.25, 1.0, 3.0), logit_scale=pick(0.5, 1.0, 4.0), loop=loop)
    p = Pair(cfg, seed=seed, exact=seed % 3 != 0, max_ctx=512, max_seqs=3, step_tokens=pick(48, 200, 512))      # (every third one in serving mode)
    ids = p.ids(170, seed)
    want = p.o.forward(ids)
    p.check(p.run_cuts(ids, []), want, "whole")
    p.check(p.run_cuts(ids, [1, 3, 40, 41, 100, 133] + list(range(140, 170))), want, "portions and decoding")
    p.close()


def test_rotary_interpolation_shows_far_beyond_the_original_length():
    # positions many times the original length: a frequency table without the interpolation, or without the factor on cos / sin, gives other logits
    sc = {"factor": 8.0, "original": 16, "fast": 1.5, "slow": 0.25}      # the ramp runs from pair 1 to pair 5 of 8
    layer = A(heads=2, dim=4, rot_dim=16, vdim=8, kv_rank=8, base=50.0, scaling=sc)
    cfg = cfg_of([layer], width=32, vocab=40)
    p = Pair(cfg, seed=15)
    ids = p.ids(300, 8)
    want = p.o.forward(ids)
    p.check(p.run_cuts(ids, [290] + list(range(291, 300))), want, "YaRN rotary")
    for other_sc in (None, dict(sc, factor=7.0), dict(sc, original=32)):
        other = Gatuzen(cfg_of([dict(layer, scaling=other_sc)], width=32, vocab=40), p.o.w).forward(ids)
        assert np.abs(other[-1] - want[-1]).max() > 50 * p.tol
    p.close()


def test_long_decoding_keeps_states_and_tails():
    cfg = cfg_of([G(heads=2, dim=16, vdim=8), M(heads=2, vdim=8, state=8, groups=1, conv=4, moe=E(3, 2, 8)), A(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=8)], width=24, vocab=40,
                 taps=4, loop=(0, 2, 2))
    p = Pair(cfg, seed=12)
    ids = p.ids(400, 9)
    p.check(p.run_cuts(ids, list(range(3, 400))), p.o.forward(ids), "397 decoded tokens")
    p.close()


def test_greedy_generation_through_the_entry_points():
    cfg = synth.gatuzen_config(**TINY)
    p = Pair(cfg, seed=13, max_seqs=4)
    prompts = [p.ids(n, 20 + i) for i, n in enumerate([9, 40, 1])]
    want = [p.o.greedy(list(pr), 10) for pr in prompts]
    for pr, w in zip(prompts, want):
        toks, usage = p.m.generate(pr, max_tokens=10)          # decoded tokens are fed back on the device: the experts' table is read there
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
    lg = p.m.forward_initial(prompts[1], 0)[0, 0]
    p.check(lg[None], p.o.forward(prompts[1])[-1:], "forward_initial")
    p.close()


def test_sampler_runs_on_the_engine():
    cfg = synth.gatuzen_config(**TINY)
    p = Pair(cfg, seed=14)
    pr = p.ids(12, 1)
    a, _ = p.m.generate(pr, max_tokens=8, temperature=0.8, top_p=0.9, top_k=20, seed=5)
    b, _ = p.m.generate(pr, max_tokens=8, temperature=0.8, top_p=0.9, top_k=20, seed=5)
    assert a == b and len(a) == 8 and all(0 <= t < cfg["vocab"] for t in a)
    p.close()
