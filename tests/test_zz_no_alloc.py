"""The allocation-free attention entry point (pe_attn_varlen_static) against the regular one.

Some callers of this library cannot hand over scratch memory and may not allocate any: a
plug-in inside a process whose allocator already owns the GPU, or a serving thread that must
not call cudaMalloc on its request path. For them the library keeps the attention tile table
in a built-in device array. This file is named to be collected last, and the test passes both
alone in a fresh process and after every other test.
"""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(lengths, n_heads, seed, device):
    gen = torch.Generator().manual_seed(seed)
    qkv = torch.randn(sum(lengths), 3 * n_heads * 64, generator=gen).to(torch.bfloat16).to(device)
    cu = torch.zeros(len(lengths) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lengths).cumsum(0)
    return qkv, cu.to(device)


def test_static_scratch_matches_caller_scratch_twice_in_a_row(pe, cuda_device):
    from flash_modernbert_b200 import _lib, ops

    # two calls in a row with different shapes and both kernel families: the second must not
    # see anything the first left in the shared table
    cases = [
        ([700, 1, 129, 64, 300, 33], 12, 64),     # tensor-memory kernel, sliding window
        ([48, 8, 30, 41, 19, 5], 4, None),        # register-tiled short kernel, full attention
        ([257, 128, 2048], 2, None),              # tensor-memory kernel, full attention
    ]
    for seed, (lengths, n_heads, window) in enumerate(cases):
        qkv, cu = _case(lengths, n_heads, seed, cuda_device)
        expected = ops.attention_varlen_qkv(qkv, cu, max(lengths), n_heads, window)
        got = ops.attention_varlen_qkv_static(qkv, cu, max(lengths), n_heads, window)
        again = ops.attention_varlen_qkv_static(qkv, cu, max(lengths), n_heads, window)
        ops.check_status(cuda_device)
        # same kernels on the same data: identical bits (the parity tests' tolerance is
        # looser: max-abs 0.03 against the fp32 reference)
        assert torch.equal(got, expected)
        assert torch.equal(again, expected)

    # sizes beyond the built-in table are refused with a clear error, nothing is launched
    lib = _lib.load()
    qkv, cu = _case([16], 1, 9, cuda_device)
    out = torch.empty(16, 64, dtype=torch.bfloat16, device=cuda_device)
    rc = lib.pe_attn_varlen_static(qkv.data_ptr(), cu.data_ptr(), 4097, 16, 1, -1, 16, out.data_ptr(),
                                   None, _lib.current_stream_ptr())
    assert rc == _lib.PE_ERR_WORKSPACE and "exceed" in _lib.last_error()
    rc = lib.pe_attn_varlen_static(qkv.data_ptr(), cu.data_ptr(), 1, (1 << 20) + 1, 1, -1, 16,
                                   out.data_ptr(), None, _lib.current_stream_ptr())
    assert rc == _lib.PE_ERR_WORKSPACE


def test_static_scratch_allocates_nothing_and_works_at_its_limits(pe, cuda_device):
    """At exactly the documented maximum (4,096 sequences, 1,048,576 tokens) the built-in table
    is large enough and the result equals the caller-scratch entry point's; one token or one
    sequence more is refused. Around direct calls through the C ABI the device's free memory and
    torch's allocation count do not move: the entry point reserves nothing."""
    from flash_modernbert_b200 import _lib, ops

    lib = _lib.load()
    lengths = [256] * 4096
    total = sum(lengths)
    assert total == 1 << 20
    qkv, cu = _case(lengths, 1, 31, cuda_device)
    out = torch.empty(total, 64, dtype=torch.bfloat16, device=cuda_device)
    status = ops.status_word(cuda_device)
    stream = _lib.current_stream_ptr()

    def call(n_seqs, tokens):
        return lib.pe_attn_varlen_static(qkv.data_ptr(), cu.data_ptr(), n_seqs, tokens, 1, 64, 256,
                                         out.data_ptr(), status.data_ptr(), stream)

    assert call(4096, total) == 0, _lib.last_error()          # first call: looks the array's address up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(cuda_device)
    allocated_before = torch.cuda.memory_allocated(cuda_device)
    out.zero_()
    assert call(4096, total) == 0 and call(4096, total) == 0
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(cuda_device)
    assert torch.cuda.memory_allocated(cuda_device) == allocated_before
    assert free_after == free_before
    ops.check_status(cuda_device)
    expected = ops.attention_varlen_qkv(qkv, cu, 256, 1, 64)
    assert torch.equal(out, expected)
    assert call(4097, total) == _lib.PE_ERR_WORKSPACE
    assert call(4096, total + 1) == _lib.PE_ERR_WORKSPACE
