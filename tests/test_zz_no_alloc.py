"""``tb200_decode_attention_static``: paged decode attention for hosts that cannot allocate
device memory (their pool owns it all, or the allocator must not be entered where they run).
Its split-KV scratch is a fixed 16 MiB array inside the library instead of a cudaMalloc.

The test calls it through the C ABI twice in a row, on different problems, and compares each
result with the regular ``decode_attention`` kernel's: the second call runs on whatever the
first one left in the shared array, so a result that depended on stale scratch would show.
It also checks that a problem whose partials cannot fit the array is refused with a message
that names the limit. Collected last on purpose (file name), and self-contained: it passes
alone in a fresh process as well as after the other tests.
"""
import numpy as np
import pytest

import oracle
from refs import paged_case, rel_err
from tessel_b200.gpu import F32, GpuError

pytestmark = pytest.mark.gpu
h, i32 = np.float16, np.int32
TOL = 2e-3


def both(gpu, q, kc, vc, table, lens, scale):
    arrays = [q, kc, vc, table, lens, np.zeros(q.shape, h), np.zeros(q.shape, h)]
    bufs = [gpu.tensor(a) for a in arrays]
    B, H, D = q.shape
    NP, P, G, _ = kc.shape
    gpu.decode_attention_static((B, H, G, D, NP, P, table.shape[1]), *bufs[:5], bufs[6], scale)
    k = gpu.kernel("decode_attention", [a.shape for a in arrays[:6]])
    gpu.launch(k, bufs[:6] + [F32(scale)])
    gpu.sync()
    regular, static = gpu.fetch(bufs[5], h, q.shape), gpu.fetch(bufs[6], h, q.shape)
    for b in bufs:
        gpu.free(b)
    return regular, static


def test_static_scratch_entry_point_matches_the_regular_kernel(gpu):
    r = oracle.Rng(77)
    cases = [
        (32, 8, 128, [700, 33, 1152, 16, 0, 2303]),   # Llama-3-8B heads: several KV splits
        (8, 2, 64, [37, 128, 300, 511]),              # benchmark configuration 1's shape, other data
    ]
    for H, G, D, lens in cases:
        q, kc, vc, table, ln, scale = paged_case(r, len(lens), H, D, 16, lens, g=G)
        regular, static = both(gpu, q, kc, vc, table, ln, scale)
        live = np.asarray(lens) > 0
        assert np.isnan(static[~live].astype(np.float32)).all() == np.isnan(regular[~live].astype(np.float32)).all()
        assert not np.isnan(static[live].astype(np.float32)).any()
        assert rel_err(static[live], regular[live]) <= TOL
        assert rel_err(static[live], oracle.decode_attention(q, kc, vc, table, ln, scale)[live]) <= TOL


def test_static_scratch_limit_is_enforced(gpu):
    # 5000 sequences x 32 heads x (128 + 2) floats = 83 MB of partials for a single split: too much.
    dummy = gpu.alloc(64)
    with pytest.raises(GpuError, match="static scratch"):
        gpu.decode_attention_static((5000, 32, 8, 128, 64, 16, 8), dummy, dummy, dummy, dummy, dummy, dummy, 0.1)
    with pytest.raises(GpuError, match="multiple of G"):
        gpu.decode_attention_static((4, 6, 4, 128, 64, 16, 8), dummy, dummy, dummy, dummy, dummy, dummy, 0.1)
    gpu.free(dummy)
