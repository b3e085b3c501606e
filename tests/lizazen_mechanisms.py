"""Each mechanism of the Lizazen decoder alone, through its part of the package (on whatever
kernel set is handed in: the PyTorch twins on the CPU, the CUDA kernels on a GPU) against its
function of the plain implementation. Inputs and weights are made so that a fault shows: the
query matrix is the key matrix with its columns rolled, so a token whose input is the rolled
input of an earlier token meets that token's key with a score far above all others; such
pairs are put just inside and just outside a window, a chunk and the kept first tokens, at
page borders, in prompts and in decoding."""

from __future__ import annotations

import torch

import plain_lizazen as plain
from mercury_b200.parts.base import PartSpec, build_part
from sisavik_mechanisms import PAGE, Stand, assert_close, rand, run_cut, tolerances

HIDDEN = 32
ROLL = 5          # W_q = W_k with its columns rolled by this many places


def double(W):
    return {k: v.double() for k, v in W.items()}


def tie_queries_to_keys(W, prefix, heads, kv_heads, rows_per_head, biased=False, normed=False):
    """W[q] from W[k]: query head h is KV head h // group with its columns rolled."""
    group = heads // kv_heads
    wk = W[prefix + "k"].view(kv_heads, rows_per_head, HIDDEN)
    W[prefix + "q"] = torch.roll(wk.repeat_interleave(group, dim=0), ROLL, dims=-1).reshape(-1, HIDDEN).clone()
    for tied, suffix in ((biased, ".b"), (normed, ".norm")):
        if tied:
            W[prefix + "q" + suffix] = (W[prefix + "k" + suffix].view(kv_heads, rows_per_head)
                                        .repeat_interleave(group, dim=0).reshape(-1).clone())


def inputs_with_a_pair(length, query, key, seed):
    """Random rows; the row at `query` is the rolled row at `key` (times 2, for a sharp score),
    so q(query) = k(key) up to the rotation."""
    x = rand((length, HIDDEN), seed)
    x[key] = 2.0 * x[key]
    if query != key:
        x[query] = torch.roll(x[key], ROLL)
    return x


def cuts_for(length, query, key):
    marks = sorted({key + 1, query, min(query + 2, length), length})
    cuts = ([length], [query] + [1] * (length - query), [b - a for a, b in zip([0] + marks, marks)],
            [2] * (length // 2) + [1] * (length % 2))
    return [[c for c in cut if c > 0] for cut in cuts]


def bfloat16_bound(spec, W, x, want, cut, kv_heads, key_dim, value_dim, window, keep):
    """What bfloat16 storage alone costs on this case: twice the error of the PyTorch twins
    (float32 arithmetic, bfloat16 between the kernels), and at least the usual tolerance.
    Scores as sharp as these tests make them turn a rounding of the keys into a visible change
    of the weights."""
    from kernel_twins import TorchOps

    stand = Stand(TorchOps(), "cpu", torch.bfloat16, window=window, keep=keep)
    part = build_part("mixer", spec)
    part.load(W, stand.setup)
    cache = stand.layer_cache(kv_heads, key_dim, value_dim)
    got = run_cut(stand, lambda rows: part.forward(rows, stand.ctx, cache(), None), x.bfloat16(), cut)
    err = float((got.double() - want).abs().max() / float(want.abs().max()))
    return max(tolerances(torch.bfloat16), 2.0 * err)


def run_attention(ops, device, dtype, spec, W, x, want, cuts, kv_heads, key_dim, value_dim, window, keep,
                  what):
    tol = tolerances(dtype)
    if dtype == torch.bfloat16:
        tol = bfloat16_bound(spec, W, x, want, cuts[0], kv_heads, key_dim, value_dim, window, keep)
    for cut in cuts:
        stand = Stand(ops, device, dtype, window=window, keep=keep)
        part = build_part("mixer", spec)
        part.load(W, stand.setup)
        cache = stand.layer_cache(kv_heads, key_dim, value_dim)
        got = run_cut(stand, lambda rows: part.forward(rows, stand.ctx, cache(), None), x.to(dtype), cut)
        assert_close(got, want, tol, f"{what} cut {cut[:3]}")
        stand.cache.check_invariants()


def weight_on(config, W, prefix, x, query, key, fn):
    """How much of the output at `query` changes when the row at `key` is replaced: large iff
    the key is seen (the test is sharp only if this tells the two apart)."""
    other = x.clone()
    other[key] = rand((HIDDEN,), 999)
    a, b = fn(x.double()), fn(other.double())
    return float((a[query] - b[query]).norm() / a[query].norm())


# ------------------------------------------------------------------------------ embedding

def check_bigram_embedding(ops, device, dtype):
    from mercury_b200.parts.embedding import BigramEmbedding

    check_bigram_case(ops, device, dtype, 61, 24, 17, 29, 3)
    check_bigram_case(ops, device, dtype, 50000, 8, 1000003, 10 ** 15 + 37, -5)     # beyond 64-bit products


def check_bigram_case(ops, device, dtype, vocab, width, buckets, mul_prev, mul_cur):
    from mercury_b200.parts.embedding import BigramEmbedding

    part = BigramEmbedding(vocab, width, "embed", "bigram", buckets, mul_prev, mul_cur)
    W = {"embed": rand((vocab, width), 1).bfloat16(), "bigram": rand((buckets + 1, width), 2).bfloat16()}
    stand = Stand(ops, device, dtype)
    part.load(W, stand.setup)
    state = torch.full((4, 1), 12345, dtype=torch.int32, device=stand.device)   # slots used before
    tokens = torch.randint(0, vocab, (40,), generator=torch.Generator().manual_seed(3)).tolist()
    want = (W["embed"].double()[torch.tensor(tokens)]
            + plain.bigram_rows(tokens, W["bigram"].double(), buckets, mul_prev, mul_cur))
    for turn, cuts in enumerate(([40], [1] * 40, [2, 1, 16, 5, 16])):
        seq = stand.open(f"e{turn}")
        outs, at = [], 0
        for n in cuts:
            entries = stand.step([(seq, n)])
            stand.ctx.batch.token_ids[:n] = torch.tensor(tokens[at:at + n], dtype=torch.int32)
            outs.append(part.forward(stand.ctx.batch.token_ids, stand.ctx, state=state).clone())
            stand.done(entries)
            at += n
        stand.cache.close(seq)
        assert_close(torch.cat(outs), want, 1e-6, f"bigram embedding cut {cuts[:3]}")
    # two sequences in one step, one at its start and one going on
    a, b = stand.open("a"), stand.open("b")
    first = stand.step([(a, 7)])
    stand.ctx.batch.token_ids[:7] = torch.tensor(tokens[:7], dtype=torch.int32)
    part.forward(stand.ctx.batch.token_ids, stand.ctx, state=state)
    stand.done(first)
    stand.step([(b, 5), (a, 4)])
    stand.ctx.batch.token_ids[:9] = torch.tensor(tokens[:5] + tokens[7:11], dtype=torch.int32)
    got = part.forward(stand.ctx.batch.token_ids, stand.ctx, state=state)
    assert_close(got[:5], want[:5], 1e-6, "bigram embedding, a new sequence in a batch")
    assert_close(got[5:9], want[7:11], 1e-6, "bigram embedding, a sequence going on in a batch")


# ------------------------------------------------------------------------------ rotation

def check_scaled_rotation(ops, device, dtype):
    """The tables of a rotation whose long wavelengths are slowed down, in all three ranges."""
    from mercury_b200.parts.rotary import RotaryEncoding

    stand = Stand(ops, device, dtype)
    for dims, base, scaling in ((16, 10000.0, {"factor": 6.0, "low": 1.0, "high": 3.0, "original": 64}),
                                (6, 50.0, {"factor": 2.0, "low": 0.5, "high": 3.0, "original": 20}),
                                (8, 300.0, None)):
        part = RotaryEncoding(dims + 4, base, dims, table_precision="float64", scaling=scaling)
        part.load({}, stand.setup)
        f = plain.rotary_frequencies(dims, base, scaling)
        if scaling:
            waves = 2 * torch.pi / torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)])
            edges = (scaling["original"] / scaling["high"], scaling["original"] / scaling["low"])
            assert (waves < edges[0]).any() and (waves > edges[1]).any()
        angle = torch.arange(200, dtype=torch.float64)[:, None] * f[None, :]
        cos, sin = part.rotary_tables()
        assert_close(cos[:200], angle.cos(), 1e-6, "scaled rotation, cosines")
        assert_close(sin[:200], angle.sin(), 1e-6, "scaled rotation, sines")


# ------------------------------------------------------------------------------ attention layers

def capped_case(heads=4, kv_heads=2, dim=16, window=21, rot=4, softcap=30.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": 2.0, "softcap": softcap,
         "mask": {"size": window}, "rot": {"base": 100.0, "dims": rot,
                                           "scaling": {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 40}}}
    W = {"a.k": rand((kv_heads * dim, HIDDEN), 10, 0.3), "a.k.b": rand((kv_heads * dim,), 12, 0.02),
         "a.k.norm": 1.0 + rand((kv_heads * dim,), 14, 0.05), "a.sink": rand((heads,), 15) + 12.0,
         "a.o": rand((HIDDEN, heads * dim), 16, 0.2), "a.o.b": rand((HIDDEN,), 17, 0.1)}
    tie_queries_to_keys(W, "a.", heads, kv_heads, dim, biased=True, normed=True)
    spec = PartSpec("masked_attention", {
        "hidden_size": HIDDEN, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": dim,
        "scale": m["scale"], "eps": 1e-6, "prefix": "a.", "mask": {"kind": "sliding", "size": window},
        "bias": ("q", "k", "o"), "values_from_keys": True, "qk_norm": "projection", "softcap": softcap,
        "sink": True, "position_encoding": PartSpec("rotary", {
            "head_dim": dim, "theta": 100.0, "rotary_dim": rot, "table_precision": "float64",
            "scaling": m["rot"]["scaling"]})})
    return m, {k: v.bfloat16() for k, v in W.items()}, spec


def check_capped_window_attention(ops, device, dtype):
    """The sink is about as large as the aligned pair's capped score, so leaving it out, or
    capping or scaling it, moves the output; the window's edge decides whether the pair meets."""
    m, W, spec = capped_case()
    window, length = m["mask"]["size"], 90
    pairs = [(70, 70 - window + 1), (70, 70 - window), (64, 64 - window + 1), (63, 48),
             (31 + window, 31), (31 + window, 32), (89, 89 - window), (47, 47)]
    for query, key in pairs:
        x = inputs_with_a_pair(length, query, key, 21 + query + key).to(dtype).float()
        fn = lambda rows: plain.capped_window_attention(rows, m, double(W), "a.", 1e-6)
        want = fn(x.double())
        if query != key:
            moved = weight_on(m, W, "a.", x, query, key, fn)
            assert (moved > 0.2) if query - key < window else (moved < 1e-9), (query, key, moved)
        run_attention(ops, device, dtype, spec, W, x, want, cuts_for(length, query, key), m["kv_heads"],
                      m["dim"], m["dim"], window, 0, f"capped attention q{query} k{key}")


def check_far_key_among_hundreds(ops, device, dtype):
    """A window of 200 keys over a prompt of 240: the one key that matters is 199 back (seen) or
    200 back (not seen), among hundreds that weigh next to nothing, in a prompt and in decoding."""
    m, W, spec = capped_case(window=200)
    window, length = 200, 240
    for query, key in ((235, 36), (235, 35), (239, 40), (216, 16)):
        x = inputs_with_a_pair(length, query, key, 300 + query + key).to(dtype).float()
        fn = lambda rows: plain.capped_window_attention(rows, m, double(W), "a.", 1e-6)
        want = fn(x.double())
        moved = weight_on(m, W, "a.", x, query, key, fn)
        assert (moved > 0.2) if query - key < window else (moved < 1e-9), (query, key, moved)
        cuts = [[length], [query - 3] + [1] * (length - query + 3), [100, 2, 77, length - 179]]
        run_attention(ops, device, dtype, spec, W, x, want, cuts, m["kv_heads"], m["dim"], m["dim"],
                      window, 0, f"far key q{query} k{key}")


def differential_case(heads=4, kv_heads=2, dim=8, vdim=24, window=21, keep=5, rot=2, diff=0.35):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": 1.2, "diff": diff,
         "mask": {"size": window, "keep_first": keep}, "rot": {"base": 100.0, "dims": rot}}
    W = {"a.k": rand((kv_heads * 2 * dim, HIDDEN), 30, 0.4), "a.v": rand((kv_heads * vdim, HIDDEN), 31, 0.3),
         "a.lq1": rand((dim,), 32, 0.3), "a.lk1": rand((dim,), 33, 0.3), "a.lq2": rand((dim,), 34, 0.3),
         "a.lk2": rand((dim,), 35, 0.3), "a.o": rand((HIDDEN, heads * vdim), 36, 0.2)}
    # map 2 is not tied as sharply as map 1, or the two maps would cancel
    tie_queries_to_keys(W, "a.", heads, kv_heads, 2 * dim)
    q = W["a.q"].view(heads, 2, dim, HIDDEN)
    q[:, 1] = rand((heads, dim, HIDDEN), 37, 0.4)
    spec = PartSpec("masked_attention", {
        "hidden_size": HIDDEN, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": dim,
        "value_dim": vdim, "scale": m["scale"], "eps": 1e-6, "prefix": "a.", "maps": 2, "diff": diff,
        "mask": {"kind": "sliding", "size": window, "keep_first": keep},
        "position_encoding": PartSpec("rotary", {"head_dim": dim, "theta": 100.0, "rotary_dim": rot,
                                                 "table_precision": "float64"})})
    return m, {k: v.bfloat16() for k, v in W.items()}, spec


def check_differential_attention(ops, device, dtype):
    m, W, spec = differential_case()
    window, keep, length = m["mask"]["size"], m["mask"]["keep_first"], 90
    pairs = [(70, 70 - window + 1), (70, 70 - window), (80, keep - 1), (80, keep), (47, 0),
             (63, 48), (31 + window, 31), (31 + window, 32), (3, 1)]
    for query, key in pairs:
        x = inputs_with_a_pair(length, query, key, 41 + query + key).to(dtype).float()
        fn = lambda rows: plain.differential_attention(rows, m, double(W), "a.", 1e-6)
        want = fn(x.double())
        moved = weight_on(m, W, "a.", x, query, key, fn)
        seen = query - key < window or key < keep
        assert (moved > 0.2) if seen else (moved < 1e-9), (query, key, moved)
        run_attention(ops, device, dtype, spec, W, x, want, cuts_for(length, query, key), m["kv_heads"],
                      2 * m["dim"], m["vdim"], window, keep, f"differential attention q{query} k{key}")


def chunked_case(heads=6, kv_heads=2, dim=8, vdim=12, chunk=21, rot=2):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": 1.5,
         "mask": {"size": chunk}, "rot": {"base": 100.0, "dims": rot}}
    W = {"a.k": rand((kv_heads * dim, HIDDEN), 50, 0.4), "a.k.b": rand((kv_heads * dim,), 51, 0.05),
         "a.v": rand((kv_heads * vdim, HIDDEN), 52, 0.3), "a.v.b": rand((kv_heads * vdim,), 53, 0.2),
         "a.o": rand((HIDDEN, heads * vdim), 54, 0.2), "a.o.b": rand((HIDDEN,), 55, 0.1)}
    tie_queries_to_keys(W, "a.", heads, kv_heads, dim, biased=True)
    spec = PartSpec("masked_attention", {
        "hidden_size": HIDDEN, "num_heads": heads, "num_kv_heads": kv_heads, "head_dim": dim,
        "value_dim": vdim, "scale": m["scale"], "eps": 1e-6, "prefix": "a.",
        "mask": {"kind": "chunked", "size": chunk}, "bias": ("q", "k", "v", "o"),
        "position_encoding": PartSpec("rotary", {"head_dim": dim, "theta": 100.0, "rotary_dim": rot,
                                                 "table_precision": "float64"})})
    return m, {k: v.bfloat16() for k, v in W.items()}, spec


def check_chunked_attention(ops, device, dtype):
    """Chunks are counted from position 0, wherever the prompt is cut: a pair on the two sides
    of a chunk's first position does not meet, however near."""
    m, W, spec = chunked_case()
    chunk, length = m["mask"]["size"], 90
    pairs = [(3 * chunk + 5, 3 * chunk), (3 * chunk + 5, 3 * chunk - 1), (4 * chunk - 1, 3 * chunk),
             (4 * chunk, 4 * chunk - 1), (2 * chunk, 2 * chunk), (chunk - 1, 0), (48, 47), (64, 63)]
    for query, key in pairs:
        x = inputs_with_a_pair(length, query, key, 61 + query + key).to(dtype).float()
        fn = lambda rows: plain.chunked_attention(rows, m, double(W), "a.")
        want = fn(x.double())
        if query != key:
            moved = weight_on(m, W, "a.", x, query, key, fn)
            assert (moved > 0.2) if query // chunk == key // chunk else (moved < 1e-9), (query, key, moved)
        run_attention(ops, device, dtype, spec, W, x, want, cuts_for(length, query, key), m["kv_heads"],
                      m["dim"], m["vdim"], chunk, 0, f"chunked attention q{query} k{key}")


# ------------------------------------------------------------------------------ retention

def check_retention(ops, device, dtype, heads=3, dim=12, vdim=20, rot=8, length=80):
    """A key far back is what a slow head still reads and a fast head has forgotten."""
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": [0.999, 0.9, 0.5][:heads] + [0.97] * (heads - 3),
         "rot": {"base": 50.0, "dims": rot}}
    W = {"a.q": rand((heads * dim, HIDDEN), 70, 0.3), "a.k": rand((heads * dim, HIDDEN), 71, 0.3),
         "a.v": rand((heads * vdim, HIDDEN), 72, 0.3), "a.g": rand((heads * vdim, HIDDEN), 73, 0.3),
         "a.o": rand((HIDDEN, heads * vdim), 74, 0.2)}
    W = {k: v.bfloat16() for k, v in W.items()}
    spec = PartSpec("retention", {
        "hidden_size": HIDDEN, "heads": heads, "key_dim": dim, "value_dim": vdim, "decay": m["decay"],
        "eps": 1e-6, "prefix": "a.", "position_encoding": PartSpec("rotary", {
            "head_dim": dim, "theta": 50.0, "rotary_dim": rot, "table_precision": "float64"}) if rot else None})
    x = rand((length, HIDDEN), 75)
    x[2] = 6.0 * x[2]                             # a loud token far back
    x = x.to(dtype).float()
    want = plain.retention(x.double(), m, double(W), "a.", 1e-6)
    stand = Stand(ops, device, dtype)
    part = build_part("mixer", spec)
    part.load(W, stand.setup)
    state = torch.zeros((4, *part.state_need().shape), dtype=torch.float32, device=stand.device)
    for turn, cuts in enumerate(([length], [length - 40] + [1] * 40, [2, 31, 1, 33, length - 67],
                                 [2] * (length // 2))):
        state.fill_(3.0)                          # slots that other requests have used
        def forward(rows):
            if stand.ctx.batch.positions[0].item() == 0:
                state[stand.ctx.batch.slots[0].item()].zero_()
            return part.forward(rows, stand.ctx, None, state)
        got = run_cut(stand, forward, x.to(dtype), cuts, name=f"r{turn}")
        assert_close(got, want, tolerances(dtype), f"retention cut {cuts[:3]}")


# ------------------------------------------------------------------------------ norms and feed-forwards

def check_join_of_two_mixers(ops, device, dtype):
    h = rand((9, 136), 3).to(device) + 5.0
    a, b = rand((9, 136), 4, 3.0).to(device), rand((9, 136), 5, 0.2).to(device)
    wa, wb, w, w2 = ((1.0 + rand((136,), 6 + i, 0.1)).to(device) for i in range(4))
    for weights, scales, follow in (((wa, wb), (0.5, 0.5), None), ((wa, wb), (0.3, 1.1), w2),
                                    ((None, None), (1.0, 1.0), w2)):
        got = h.clone()
        out = torch.empty((9, 136), dtype=dtype, device=device) if follow is not None else None
        ops.rmsnorm_join_add(got, a, b, weights[0], weights[1], scales[0], scales[1], w, 1e-5, follow,
                             1e-4, out)
        x, y = a.double().cpu(), b.double().cpu()
        if weights[0] is not None:
            x, y = plain.rms_norm(x, wa.double().cpu(), 1e-5), plain.rms_norm(y, wb.double().cpu(), 1e-5)
        want = h.double().cpu() + plain.rms_norm(scales[0] * x + scales[1] * y, w.double().cpu(), 1e-5)
        assert_close(got, want, 1e-6, "join of two mixers")
        if follow is not None:
            assert_close(out, plain.rms_norm(want, w2.double().cpu(), 1e-4),
                         1e-6 if dtype == torch.float32 else 8e-3, "the norm computed ahead")


def check_clamped_feed_forward(ops, device, dtype, ff=40, limit=0.6):
    """Gate and up values beyond the limit on both sides, so each clamp (and the missing lower
    clamp of the gate) shows."""
    W = {"f.gate": rand((ff, HIDDEN), 80, 0.4), "f.up": rand((ff, HIDDEN), 81, 0.4),
         "f.down": rand((HIDDEN, ff), 82, 0.2)}
    W = {k: v.bfloat16() for k, v in W.items()}
    stand = Stand(ops, device, dtype)
    part = build_part("feed_forward", PartSpec("gated", {
        "hidden_size": HIDDEN, "intermediate_size": ff, "prefix": "f.", "activation": "clamped_sigmoid",
        "limit": limit, "slope": 1.702, "names": ("gate", "up", "down")}))
    part.load(W, stand.setup)
    x = rand((21, HIDDEN), 83).to(dtype)
    raw = x.double() @ W["f.gate"].double().T
    assert (raw > limit).any() and (raw < -limit).any()
    want = plain.dense_feed_forward(x.double(), {"limit": limit}, double(W), "f.")
    seq = stand.open("f")
    stand.step([(seq, 21)])
    got = part.forward(x.to(stand.device), stand.ctx)
    assert_close(got, want, tolerances(dtype), "clamped feed-forward")


def check_experts_weighted_on_their_input(ops, device, dtype, experts=5, top=2, ff=24, shared=16):
    mlp = {"router": {"experts": experts, "top": top}, "expert": {"ff": ff}, "shared": {"ff": shared}}
    W = {"f.router": rand((experts, HIDDEN), 90, 0.2), "f.shared.gate": rand((shared, HIDDEN), 91, 0.3),
         "f.shared.up": rand((shared, HIDDEN), 92, 0.3), "f.shared.down": rand((HIDDEN, shared), 93, 0.2)}
    for e in range(experts):
        W[f"f.e{e}.gate"] = rand((ff, HIDDEN), 100 + 3 * e, 0.4)
        W[f"f.e{e}.up"] = rand((ff, HIDDEN), 101 + 3 * e, 0.4)
        W[f"f.e{e}.down"] = rand((HIDDEN, ff), 102 + 3 * e, 0.2)
    W = {k: v.bfloat16() for k, v in W.items()}
    stand = Stand(ops, device, dtype)
    part = build_part("feed_forward", PartSpec("routed_experts", {
        "hidden_size": HIDDEN, "intermediate_size": ff, "experts": experts, "top": top,
        "route_scale": 1.0, "prefix": "f.", "correction": False, "weight_on": "input",
        "shared": PartSpec("gated", {"hidden_size": HIDDEN, "intermediate_size": shared,
                                     "prefix": "f.shared.", "activation": "silu",
                                     "names": ("gate", "up", "down"), "float_out": True,
                                     "out_name": "shared_out"})}))
    part.load(W, stand.setup)
    x = rand((37, HIDDEN), 94).to(dtype)
    want = plain.routed_feed_forward(x.double(), mlp, double(W), "f.")
    # weighting the output instead would give something else
    scores = torch.sigmoid(x.double() @ W["f.router"].double().T)
    assert float((scores.topk(top).values - 1.0).abs().min()) > 1e-3
    seq = stand.open("f")
    stand.step([(seq, 37)])
    routed, common = part.forward(x.to(stand.device), stand.ctx)
    assert_close(routed.double().cpu() + common.double().cpu(), want, tolerances(dtype),
                 "experts weighted on their input")


ALL = [check_bigram_embedding, check_scaled_rotation, check_capped_window_attention,
       check_far_key_among_hundreds,
       check_differential_attention, check_chunked_attention, check_retention,
       check_join_of_two_mixers, check_clamped_feed_forward, check_experts_weighted_on_their_input]
