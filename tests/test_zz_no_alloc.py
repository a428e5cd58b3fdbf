"""The allocation-free top-k entry point (dsa_topk_select_static).

Some hosts of this library cannot allocate device memory for scratch: an
inference runtime that freezes its memory pool before serving, a plugin that only
ever sees its input and output buffers, code that runs while a CUDA graph is
being captured. For them the library carries a fixed 4 MiB scratch array of its
own. This test calls that entry point through the C ABI and checks that it
returns exactly what the regular entry point (caller-owned scratch) returns, on
two calls in a row with different shapes, so that the second call meets whatever
the first one left behind in the shared array. Collected last on purpose: a run
that stops at the first failure has then already run every other test.
"""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _static_topk(lib, logits, seq_lens, topk, pad, offset, want_vals=True):
    R, n = logits.shape
    out_idx = torch.empty(R, topk, dtype=torch.int32, device=logits.device)
    out_val = torch.empty(R, topk, dtype=torch.float32, device=logits.device) if want_vals else None
    rc = lib.dsa_topk_select_static(
        logits.data_ptr(), None if seq_lens is None else seq_lens.data_ptr(), out_idx.data_ptr(),
        None if out_val is None else out_val.data_ptr(), R, n, logits.stride(0), topk, pad, offset,
        torch.cuda.current_stream().cuda_stream)
    return rc, out_idx, out_val


def test_static_scratch_topk_matches_regular_entry_point():
    from dsa_multi_layer_indexer_b200 import _lib, ops

    lib = _lib.lib()
    torch.manual_seed(0)
    # Rows longer than 262144 logits are the ones that use the built-in scratch. Call 1: one long
    # row; call 2: a longer ragged row with ties, laid out differently in the scratch; call 3: two
    # rows for the 16-CTA cluster kernel and call 4 three short ones for the 1-8-CTA form, neither of
    # which uses the scratch or minds the leftovers.
    cases = [
        (torch.randn(1, 300000, device="cuda"), None, 2048),
        ((torch.randint(-6, 6, (1, 450000), device="cuda").float() * 0.5).contiguous(),
         torch.tensor([440001], dtype=torch.int32, device="cuda"), 2048),
        ((torch.randint(-6, 6, (2, 150000), device="cuda").float() * 0.5).contiguous(),
         torch.tensor([150000, 140001], dtype=torch.int32, device="cuda"), 2048),
        ((torch.randint(-6, 6, (3, 40000), device="cuda").float() * 0.5).contiguous(),
         torch.tensor([40000, 1500, 17], dtype=torch.int32, device="cuda"), 2048),
    ]
    for logits, lens, k in cases:
        rc, idx, val = _static_topk(lib, logits, lens, k, pad=-1, offset=7)
        assert rc == 0, lib.dsa_last_error()
        want_idx, want_val = ops.topk_select(logits, k, lens, pad_value=-1, index_offset=7, return_values=True)
        torch.cuda.synchronize()
        assert torch.equal(idx, want_idx)
        assert torch.equal(val, want_val)
    # the same first case again: the array now holds the second call's leftovers
    logits, lens, k = cases[0]
    rc, idx, _ = _static_topk(lib, logits, lens, k, pad=-1, offset=0, want_vals=False)
    assert rc == 0
    assert torch.equal(idx, ops.topk_select(logits, k, lens, pad_value=-1))
    _lib.check_device_status()


def test_static_scratch_topk_rejects_what_does_not_fit():
    from dsa_multi_layer_indexer_b200 import _lib

    lib = _lib.lib()
    logits = torch.zeros(2, 300000, device="cuda")  # 2 rows of 300000 need more scratch than the 4 MiB the array holds
    rc, _, _ = _static_topk(lib, logits, None, 2048, pad=-1, offset=0)
    assert rc == -2
    msg = lib.dsa_last_error().decode()
    assert "scratch" in msg and "4194304" in msg
