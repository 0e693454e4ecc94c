"""The allocation-free argmax entry (collected last: the file name sorts after every other test file).

Some callers of the library cannot allocate device memory -- a plugin handed only one call's tensors, or code running
where cudaMalloc is off limits -- so wein_b200_argmax_rows_noalloc keeps its slice maxima in an array built into the
library.  It must give exactly the tokens of wein_b200_argmax_rows (integer output: bit-exact), on two calls in a row
(the second call finds the previous call's words in the shared array), alone or after the rest of the suite."""
import numpy as np
import pytest
import torch

from oracle import oracle as orc
from tests.gpu_util import dev, host, rand_bf16

pytestmark = pytest.mark.gpu


def test_noalloc_argmax_matches_scratch_entry_twice():
    from inferulm_b200 import ops
    from inferulm_b200.lib import WeinB200Error
    n = 151936
    for call, (s, seed) in enumerate(((7, 1), (4, 2))):
        rs = np.random.default_rng(seed)
        x = rand_bf16(rs, s * n, 3.0).reshape(s, n)
        x[0, 5] = x[0, 90000] = orc.f32_to_bf16(np.array([40.0], np.float32))[0]   # a tie: the lower index wins
        rows = np.arange(s, dtype=np.uint32)[::-1].copy()
        xd, rd = dev(x.reshape(-1)), dev(rows)
        want = torch.empty(s, dtype=torch.int32, device="cuda")
        scratch = torch.empty(s * ops.ARGMAX_SPLIT, dtype=torch.int64, device="cuda")
        ops.argmax_rows(xd, rd, scratch, want, n, s)
        got = torch.full((s,), -1, dtype=torch.int32, device="cuda")
        ops.argmax_rows_noalloc(xd, rd, got, n, s)
        torch.cuda.synchronize()
        assert np.array_equal(host(got, np.uint32), host(want, np.uint32)), call
        assert host(got, np.uint32)[-1] == 5                                       # rows[-1] == 0, the tied row
        assert np.array_equal(host(got, np.uint32), orc.argmax_rows(x.reshape(-1), rows, n, threads=4)), call
    # the capacity edge: 256 rows fill the built-in array to its last word (row 255's slices sit at words 8160..8191)
    s, n2 = ops.ARGMAX_NOALLOC_MAX_ROWS, 4099
    rs = np.random.default_rng(3)
    x = rand_bf16(rs, s * n2, 3.0)
    rows = rs.permutation(s).astype(np.uint32)
    xd, rd = dev(x), dev(rows)
    want = torch.empty(s, dtype=torch.int32, device="cuda")
    scratch = torch.empty(s * ops.ARGMAX_SPLIT, dtype=torch.int64, device="cuda")
    ops.argmax_rows(xd, rd, scratch, want, n2, s)
    got = torch.full((s,), -1, dtype=torch.int32, device="cuda")
    ops.argmax_rows_noalloc(xd, rd, got, n2, s)
    torch.cuda.synchronize()
    assert np.array_equal(host(got, np.uint32), host(want, np.uint32))
    assert np.array_equal(host(got, np.uint32), orc.argmax_rows(x, rows, n2, threads=4))
    # an empty call is accepted and touches nothing
    keep = got.clone()
    ops.argmax_rows_noalloc(xd, rd, got, n2, 0)
    torch.cuda.synchronize()
    assert torch.equal(got, keep)
    # beyond the built-in capacity the call is refused before any launch
    big = ops.ARGMAX_NOALLOC_MAX_ROWS + 1
    z = torch.zeros(big * 8, dtype=torch.int16, device="cuda")
    with pytest.raises(WeinB200Error) as ei:
        ops.argmax_rows_noalloc(z, dev(np.arange(big, dtype=np.uint32)), torch.zeros(big, dtype=torch.int32, device="cuda"), 8, big)
    assert ei.value.code == -4
