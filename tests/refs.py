"""Plain f64 procedures the reference's own tests check its kernels against
(tests/common/mod.rs:45-173), restated in numpy, and the reference's closeness
rule (tests/common/mod.rs:37-43). Test infrastructure only."""
import numpy as np


def assert_close(what, got, want, tol):
    got = np.asarray(got, np.float32).reshape(-1)
    want = np.asarray(want, np.float32).reshape(-1)
    assert got.shape == want.shape, what
    assert not np.isnan(got).any(), f"{what}: NaN"
    d = float(np.abs(got - want).max()) if got.size else 0.0
    s = float(np.abs(want).max()) if want.size else 0.0
    assert d <= tol * max(s, 1.0), f"{what}: max |diff| {d} (largest {s}, tolerance {tol})"


def rel_err(got, want):
    """max |got - want| / max |want|: the metric of tests/llm.rs:20-23."""
    got = np.asarray(got, np.float64).reshape(-1)
    want = np.asarray(want, np.float64).reshape(-1)
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


def matmul_ref(a, b, bt):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return (a @ (b.T if bt else b)).astype(np.float32)


def rmsnorm_ref(x, w, eps):
    x = np.asarray(x, np.float64)
    ms = (x * x).sum(1, keepdims=True) / x.shape[1]
    return (x / np.sqrt(ms + np.float64(np.float32(eps))) * np.asarray(w, np.float64)[None, :]).astype(np.float32)


def attention_ref(q, k, v, scale, starts=None):
    """Causal attention per head; q, k, v [h, s, d] (f64 softmax). `starts[i]`: first key row i may see."""
    q, k, v = (np.asarray(t, np.float64) for t in (q, k, v))
    h, s, d = q.shape
    o = np.zeros((h, s, d))
    for hh in range(h):
        sc = (q[hh] @ k[hh].T) * np.float64(np.float32(scale))
        for i in range(s):
            lo = 0 if starts is None else int(starts[i])
            row = sc[i, lo:i + 1]
            e = np.exp(row - row.max())
            o[hh, i] = (e[:, None] * v[hh, lo:i + 1]).sum(0) / e.sum()
    return o.astype(np.float32)


def paged_ref(q, kc, vc, table, lens, scale, G=None):
    """Decode attention in f64 (tests/common/mod.rs:140-161), grouped-query when G < H."""
    q, kc, vc = (np.asarray(t, np.float64) for t in (q, kc, vc))
    B, H, D = q.shape
    NP, P, Gk, _ = kc.shape
    o = np.full((B, H, D), np.nan)
    for b in range(B):
        n = int(lens[b])
        if n == 0:
            continue
        pages = [int(table[b, t // P]) for t in range(n)]
        offs = [t % P for t in range(n)]
        for h in range(H):
            g = h // (H // Gk)
            kk = kc[pages, offs, g]
            vv = vc[pages, offs, g]
            sc = (kk @ q[b, h]) * np.float64(np.float32(scale))
            e = np.exp(sc - sc.max())
            o[b, h] = (e[:, None] * vv).sum(0) / e.sum()
    return o.astype(np.float32)


def paged_case(rng, b, h, d, p, lens, g=None):
    """The reference's paged-attention case builder (tests/common/mod.rs:119-173): scrambled
    page order drawn from the same generator; `g` kv heads (default h)."""
    g = g or h
    mp = max(max(-(-l // p) for l in lens), 1)
    npages = sum(-(-l // p) for l in lens) + 3
    q = rng.tensor(np.float16, (b, h, d))
    kc = rng.tensor(np.float16, (npages, p, g, d))
    vc = rng.tensor(np.float16, (npages, p, g, d))
    order = list(range(npages))
    for i in range(npages - 1, 0, -1):
        u = rng.uniform(1)[0]
        j = int(np.float32((u + np.float32(1.0)) * np.float32(0.5)) * np.float32(i + 1)) % (i + 1)
        order[i], order[j] = order[j], order[i]
    table = np.zeros((b, mp), np.int32)
    nxt = 0
    for s in range(b):
        for n in range(-(-lens[s] // p)):
            table[s, n] = order[nxt]
            nxt += 1
    scale = np.float32(1.0) / np.sqrt(np.float32(d))
    return q, kc, vc, table, np.asarray(lens, np.int32), float(scale)
