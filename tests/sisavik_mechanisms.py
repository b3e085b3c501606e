"""Each mechanism of the Sisavik decoder alone, through its part of the package (on whatever
kernel set is handed in: the PyTorch twins on the CPU, the CUDA kernels on a GPU) against its
function of the plain implementation. Inputs and weights are made so that a fault shows: a
key that dominates the sum is put just inside and just outside a window, among the kept first
tokens and right behind them, at page borders, in prompts and in decoding."""

from __future__ import annotations

import torch

import plain_sisavik as plain
from mercury_b200.cache import CacheManager
from mercury_b200.engine.batch import BatchBuffers, StepEntry
from mercury_b200.engine.runner import StepContext, Workspace
from mercury_b200.parts import PartSetup
from mercury_b200.parts.base import LayerCache, PartSpec, build_part

PAGE = 16


class Stand:
    """A step context for one part: sequences, pages and slots from the cache manager."""

    def __init__(self, ops, device, dtype, window=0, keep=0, pages=24, max_tokens=256):
        self.device, self.dtype, self.ops = torch.device(device), dtype, ops
        self.setup = PartSetup(self.device, dtype, ops, 1024)
        self.cache = CacheManager([window], pages, PAGE, 4, keep_first=[keep])
        self.buffers = BatchBuffers(self.device, max_tokens, 4, 64, 1, pin=self.device.type == "cuda")
        self.ctx = StepContext(ops, Workspace(self.device, dtype, max_tokens), PAGE, dtype)
        self.pages = pages

    def open(self, name):
        return self.cache.open(name)

    def step(self, pairs):
        """pairs: [(sequence, number of new tokens)]; books the tokens before as computed."""
        entries = []
        for seq, n in pairs:
            assert self.cache.ensure(seq, seq.num_computed + n)
            entries.append(StepEntry(seq, [0] * n, []))
        self.ctx.batch = self.buffers.build(entries, PAGE)
        self.ctx.side = 0
        return entries

    def done(self, entries):
        for e in entries:
            self.cache.advance(e.seq, e.seq.num_computed + len(e.tokens))

    def layer_cache(self, kv_heads, key_dim, value_dim=None, shared=False):
        k = torch.full((self.pages, kv_heads, PAGE, key_dim), float("nan"), dtype=self.dtype,
                       device=self.device)
        v = k if shared else torch.full((self.pages, kv_heads, PAGE, value_dim or key_dim),
                                        float("nan"), dtype=self.dtype, device=self.device)
        return lambda: LayerCache(k, v, PAGE, self.ctx.batch.tables[0], True)


def rand(shape, seed, scale=1.0):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(shape, generator=gen) * scale


def assert_close(got, want, tol, what):
    got, want = got.detach().double().cpu(), want.double()
    assert torch.isfinite(got).all(), f"{what}: non-finite"
    err = float((got - want).abs().max() / max(float(want.abs().max()), 1e-9))
    assert err <= tol, f"{what}: relative error {err:.3e} > {tol:.0e}"


def run_cut(stand, forward, x, cuts, name="s"):
    """Feeds the rows of x through `forward(rows)` in steps of `cuts` tokens (one sequence);
    returns the outputs of all rows."""
    seq = stand.open(name)
    outs, at = [], 0
    for n in cuts:
        entries = stand.step([(seq, n)])
        outs.append(forward(x[at:at + n].to(stand.device)).clone())
        stand.done(entries)
        at += n
    assert at == x.shape[0]
    stand.cache.close(seq)
    return torch.cat(outs)


def tolerances(dtype):
    return 2e-5 if dtype == torch.float32 else 2e-2


# ------------------------------------------------------------------------------ the convolution

def check_short_convolution(ops, device, dtype, taps=4, width=40):
    from mercury_b200.parts.convolution import InputConvolution

    stand = Stand(ops, device, dtype)
    part = InputConvolution(width, taps, "c")
    w = rand((width, taps), 1, 0.5).bfloat16()
    part.load({"c": w}, stand.setup)
    need = part.state_need()
    state = None
    if need is not None:
        state = torch.full((4, *need.shape), float("nan"), dtype=need.dtype, device=stand.device)
    x = rand((45, width), 2)
    want = plain.short_convolution(x.double(), w.double())
    for cuts in ([45], [1] * 45, [2, 1, 3, 7, 1, 1, 16, 2, 12], [taps - 1 or 1, 45 - (taps - 1 or 1)]):
        if state is not None:
            state.fill_(float("nan"))          # a slot that another request has used
            state[:, :, :] = 7.0
        def forward(rows, state=state):
            slot_state = state
            if state is not None and stand.ctx.batch.positions[0].item() == 0:
                state[stand.ctx.batch.slots[0].item()].zero_()    # what opening a request does
            return part.forward(rows.float(), stand.ctx, slot_state)
        got = run_cut(stand, forward, x, cuts)
        # the sum is float32; its result is rounded to the activation type
        assert_close(got, want, 1e-6 if dtype == torch.float32 else 8e-3, f"convolution cut {cuts[:4]}")


# ------------------------------------------------------------------------------ norm of two mixers

def check_pair_norm(ops, device, dtype):
    h = rand((9, 136), 3).to(device) + 5.0
    a, b = rand((9, 136), 4, 3.0).to(device), rand((9, 136), 5, 0.2).to(device)
    w = (1.0 + rand((136,), 6, 0.1)).to(device)
    for second, scales in ((b, (0.6, 1.7)), (None, (0.5, 0.0))):
        got = h.clone()
        ops.rmsnorm_add(got, a, w, 1e-5, None, 0.0, None, delta2=second, scale=scales[0], scale2=scales[1])
        d = scales[0] * a.double().cpu() + (scales[1] * second.double().cpu() if second is not None else 0)
        want = h.double().cpu() + plain.rms(d, 1e-5) * w.double().cpu()
        assert_close(got, want, 1e-6, "norm behind two mixers")


# ------------------------------------------------------------------------------ sigmoid attention

def sigmoid_case(heads=4, kv_heads=2, dim=16, hidden=32, window=21, keep=5, rot=2):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": 4.0,
         "mask": {"size": window, "keep_first": keep}, "rot": {"base": 100.0, "dims": rot}}
    wk = rand((kv_heads * dim, hidden), 10, 0.3)
    wq = wk.view(kv_heads, 1, dim, hidden).expand(kv_heads, heads // kv_heads, dim, hidden)
    W = {"a.q": wq.reshape(heads * dim, hidden).clone(), "a.k": wk,
         "a.q.b": rand((heads * dim,), 11, 0.02), "a.k.b": rand((kv_heads * dim,), 12, 0.02),
         "a.q.norm": 1.0 + rand((dim,), 13, 0.05), "a.k.norm": 1.0 + rand((dim,), 14, 0.05),
         "a.pb": torch.full((heads,), -40.0) + rand((heads,), 15), "a.o": rand((hidden, heads * dim), 16, 0.2)}
    return m, {k: v.bfloat16() for k, v in W.items()}


def check_sigmoid_attention(ops, device, dtype):
    """Queries and keys come from the same matrix, so two tokens with the same input row meet
    with a score far above the (very negative) head bias and every other pair far below: the
    output at the later one doubles when the earlier one is seen."""
    m, W = sigmoid_case()
    window, keep = m["mask"]["size"], m["mask"]["keep_first"]
    spec = PartSpec("sigmoid_attention", {
        "hidden_size": 32, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
        "scale": m["scale"], "eps": 1e-6, "prefix": "a.", "window": window, "keep_first": keep,
        "position_encoding": PartSpec("rotary", {"head_dim": m["dim"], "theta": 100.0, "rotary_dim": 2,
                                                 "table_precision": "float64", "pairing": "interleaved"})})
    length = 90
    special = rand((32,), 20, 2.0)
    # (position of the query, position of the key): inside and outside the window, the last
    # kept token and the first that is not kept, page borders (16, 32, 48, 64)
    pairs = [(70, 70 - window + 1), (70, 70 - window), (64, 64 - window + 1), (63, 48), (80, keep - 1),
             (80, keep), (47, 0), (31 + window, 31), (31 + window, 32), (89, 89 - window)]
    for query, key in pairs:
        x = rand((length, 32), 21 + query + key)
        x[key] = special
        x[query] = special
        x = x.to(dtype)
        want = plain.sigmoid_attention({k: v.double() for k, v in W.items()}, "a.", m, x.double(), 1e-6)
        seen = key <= query and (query - key < window or key < keep)
        marks = sorted({key + 1, query, min(query + 2, length), length})
        for cuts in ([length], [query] + [1] * (length - query),
                     [b - a for a, b in zip([0] + marks, marks)]):
            cuts = [c for c in cuts if c > 0]
            stand = Stand(ops, device, dtype, window=window, keep=keep)
            part = build_part("mixer", spec)
            part.load(W, stand.setup)
            cache = stand.layer_cache(m["kv_heads"], m["dim"])
            got = run_cut(stand, lambda rows: part.forward(rows, stand.ctx, cache(), None), x, cuts)
            assert_close(got, want, tolerances(dtype), f"sigmoid attention q{query} k{key} cut {cuts[:3]}")
            # the special key counts twice, once, or the test is not sharp
            alone = plain.sigmoid_attention({k: v.double() for k, v in W.items()}, "a.", m,
                                            x.double()[query:query + 1], 1e-6)[0]
            ratio = float(want[query].norm() / alone.norm())
            assert (ratio > 1.6) if (seen and key != query) else (ratio < 1.4), (query, key, ratio)
            stand.cache.check_invariants()


# ------------------------------------------------------------------------------ latent attention

def latent_case(heads=3, dim=8, rot_dim=4, vdim=12, rank=20, q_rank=10, hidden=32, window=19):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank,
         "scale": 0.9, "mask": {"size": window}, "rot": {"base": 50.0, "dims": rot_dim}}
    W = {"a.dq": rand((q_rank, hidden), 30, 0.3), "a.dq.norm": 1.0 + rand((q_rank,), 31, 0.1),
         "a.uq": rand((heads * (dim + rot_dim), q_rank), 32, 0.6),
         "a.dkv": rand((rank + rot_dim, hidden), 33, 0.3), "a.dkv.norm": 1.0 + rand((rank,), 34, 0.1),
         "a.uk": rand((heads * dim, rank), 35, 0.5), "a.uv": rand((heads * vdim, rank), 36, 0.3),
         "a.o": rand((hidden, heads * vdim), 37, 0.2)}
    return m, {k: v.bfloat16() for k, v in W.items()}


def check_latent_attention(ops, device, dtype, own_window=19, cache_window=19):
    m, W = latent_case(window=own_window)
    spec = PartSpec("latent_attention", {
        "hidden_size": 32, "num_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
        "rank": m["kv_rank"], "scale": m["scale"], "eps": 1e-6, "prefix": "a.", "sink": False,
        "q_rank": m["q_rank"], "rot_dim": m["rot_dim"], "window": own_window, "cache_window": cache_window,
        "position_encoding": PartSpec("rotary", {"head_dim": m["rot_dim"], "theta": 50.0,
                                                 "rotary_dim": m["rot_dim"], "table_precision": "float64",
                                                 "pairing": "interleaved"})})
    x = rand((70, 32), 40).to(dtype)
    Wd = {k: v.double() for k, v in W.items()}
    want = plain.latent_attention(Wd, "a.", m, x.double(), 1e-6,
                                  plain.latent_rows(Wd, "a.", m, x.double(), 1e-6))
    for cuts in ([70], [33] + [1] * 37, [2, 5, 16, 1, 9, 30, 7]):
        stand = Stand(ops, device, dtype, window=cache_window)
        part = build_part("mixer", spec)
        part.load(W, stand.setup)
        cache = stand.layer_cache(1, m["kv_rank"] + m["rot_dim"], shared=True)
        got = run_cut(stand, lambda rows: part.forward(rows, stand.ctx, cache(), None), x, cuts)
        assert_close(got, want, tolerances(dtype), f"latent attention cut {cuts[:3]}")


def check_window_edge_over_cached_rows(ops, device, dtype, row=24, heads=3, window=21):
    """The attention over cached rows alone: one row is a large multiple of the query, so the
    softmax is that row when it is seen and something else when it is not."""
    from types import SimpleNamespace

    length = 75
    for query, key in ((70, 70 - window + 1), (70, 70 - window), (64, 48), (64, 43), (74, 74 - window + 1)):
        rows = rand((length, row), 50 + key, 0.3)
        q = rand((heads, row), 51)
        rows[key] = 6.0 * q[0] / q[0].norm()
        rows, q = rows.to(dtype), q.to(dtype)
        scores = (q.double() @ rows.double()[:query + 1].T) * 1.5
        seen = (query - torch.arange(query + 1)) < window
        weights = torch.softmax(scores.masked_fill(~seen[None], float("-inf")), -1)
        want = (weights @ rows.double()[:query + 1]).reshape(-1)
        stand = Stand(ops, device, dtype, window=window)
        seq = stand.open("w")
        entries = stand.step([(seq, query)])
        cache = stand.layer_cache(1, row, shared=True)()
        # fill the pages of the tokens before the query by hand, then run the query alone
        table = stand.ctx.batch.tables[0][0].tolist()
        for p in range(query):
            cache.k[table[p // PAGE], 0, p % PAGE] = rows[p].to(stand.device)
        stand.done(entries)
        entries = stand.step([(seq, 1)])
        cache = LayerCache(cache.k, cache.k, PAGE, stand.ctx.batch.tables[0], True)
        table = stand.ctx.batch.tables[0][0].tolist()
        cache.k[table[query // PAGE], 0, query % PAGE] = rows[query].to(stand.device)
        out = torch.empty((1, heads * row), dtype=dtype, device=stand.device)
        ops.paged_attention(q.reshape(1, -1).to(stand.device), heads, 1, row, stand.ctx.batch, cache, 1.5,
                            window, out)
        assert_close(out[0], want, tolerances(dtype), f"window edge q{query} k{key}")
        stand.cache.close(seq)


# ------------------------------------------------------------------------------ delta rule

def delta_case(heads=3, dim=12, rank=5, hidden=32):
    m = {"heads": heads, "dim": dim, "decay_rank": rank}
    n = heads * dim
    W = {"a.r": rand((n, hidden), 60, 0.3), "a.k": rand((n, hidden), 61, 0.3), "a.v": rand((n, hidden), 62, 0.3),
         "a.g": rand((n, hidden), 63, 0.3), "a.a": rand((n, hidden), 64, 0.3), "a.a.b": rand((n,), 65, 0.5),
         "a.w1": rand((rank, hidden), 66, 0.3), "a.w2": rand((n, rank), 67, 0.8), "a.w0": rand((n,), 68, 1.0),
         "a.norm": 1.0 + rand((n,), 69, 0.1), "a.o": rand((hidden, n), 70, 0.2)}
    return m, {k: v.bfloat16() for k, v in W.items()}


def check_generalized_delta_rule(ops, device, dtype, heads=3, dim=12, length=80):
    m, W = delta_case(heads, dim)
    spec = PartSpec("generalized_delta_rule", {"hidden_size": 32, "heads": heads, "key_dim": dim,
                                               "decay_rank": m["decay_rank"], "eps": 1e-6, "prefix": "a."})
    x = rand((length, 32), 71).to(dtype)
    want = plain.generalized_delta_rule({k: v.double() for k, v in W.items()}, "a.", m, x.double(), 1e-6)
    stand = Stand(ops, device, dtype)
    part = build_part("mixer", spec)
    part.load(W, stand.setup)
    state = torch.zeros((4, *part.state_need().shape), dtype=torch.float32, device=stand.device)
    for turn, cuts in enumerate(([length], [length - 40] + [1] * 40, [2, 31, 1, 33, length - 67])):
        state.fill_(3.0)                       # slots that other requests have used
        def forward(rows):
            if stand.ctx.batch.positions[0].item() == 0:
                state[stand.ctx.batch.slots[0].item()].zero_()
            return part.forward(rows, stand.ctx, None, state)
        got = run_cut(stand, forward, x, cuts, name=f"d{turn}")
        assert_close(got, want, tolerances(dtype), f"delta rule cut {cuts[:3]}")


# ------------------------------------------------------------------------------ rotation

def check_rotation_of_pairs(ops, device, dtype):
    """Neighbouring features are paired, and only the first numbers of a row turn."""
    from types import SimpleNamespace

    tokens, heads, row, offset, dims = 7, 3, 14, 4, 6
    positions = torch.tensor([0, 1, 5, 17, 100, 3, 999], dtype=torch.int32)
    q = rand((tokens, heads * row), 80).to(dtype)
    i = torch.arange(dims // 2, dtype=torch.float64)
    angle = torch.arange(1024, dtype=torch.float64)[:, None] * 300.0 ** (-2.0 * i / dims)
    tables = (torch.cos(angle).float().to(device), torch.sin(angle).float().to(device))
    batch = SimpleNamespace(positions=positions.to(device),
                            seq_of_token=torch.zeros(tokens, dtype=torch.int32, device=device))
    got = q.clone().to(device)
    ops.rope_rows(got, heads, row, offset, dims, tables, "interleaved", batch)
    view = q.double().view(tokens, heads, row)
    want = view.clone()
    want[..., offset:offset + dims] = plain.rotate_pairs(view[..., offset:offset + dims], positions, 300.0, dims)
    assert_close(got, want.reshape(tokens, -1), 1e-6 if dtype == torch.float32 else 8e-3, "rotation of pairs")


ALL = [check_short_convolution, check_pair_norm, check_sigmoid_attention, check_latent_attention,
       check_window_edge_over_cached_rows, check_generalized_delta_rule, check_rotation_of_pairs]
