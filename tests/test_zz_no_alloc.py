"""The entry point that allocates nothing (`tuff_argmax_noalloc`, csrc/argmax_noalloc.cu).

Some hosts of this library cannot let it call cudaMalloc: their process gave the whole GPU to an
arena of its own at start, or they sit in a loop where cudaMalloc's device-wide synchronisation
is not acceptable.  For them the greedy token choice exists in a form whose working memory is a
fixed array inside the library.  This test calls it the way such a host would — through the
exported C symbol, with raw device pointers — twice in a row on the same working array, and
wants the same tokens as the engine's ordinary argmax.  It lives in a file that pytest collects
last, so a run that stops at the first failure has seen every other test first.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from tuff_b200.kernels.build import load_library
    lib = load_library("argmax_noalloc")
    lib.tuff_argmax_noalloc.restype = ctypes.c_int
    lib.tuff_argmax_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    lib.tuff_argmax_noalloc_message.restype = ctypes.c_char_p
    return lib


def _call(lib, logits, out):
    return lib.tuff_argmax_noalloc(logits.data_ptr(), logits.shape[0], logits.shape[1], out.data_ptr(),
                                   torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("rows,V", [(8, 65536), (3, 301), (256, 1000)])
def test_same_tokens_as_the_ordinary_argmax_twice_in_a_row(rows, V):
    from tuff_b200.kernels import ops
    lib = _lib()
    rng = np.random.default_rng(rows + V)
    for call in range(2):                                   # the second call finds the first one's leftovers
        host = rng.normal(size=(rows, V)).astype(np.float32)
        host[0, [V // 3, V - 1]] = 9.0                      # a tie: the lower index must win
        if rows > 1:
            host[1, :] = -2.5                               # all equal: token 0
        logits = torch.from_numpy(host).cuda()
        want = torch.empty(rows, dtype=torch.int32, device="cuda")
        ops.argmax(logits, want)                            # the existing entry point
        got = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
        allocated = torch.cuda.memory_allocated()
        rc = _call(lib, logits, got)
        assert rc == 0, lib.tuff_argmax_noalloc_message(rc).decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == allocated   # nothing was taken from torch's allocator either
        assert got.tolist() == want.tolist() == [int(r.argmax()) for r in host]
        assert got[0].item() == V // 3 and (rows == 1 or got[1].item() == 0)


def test_refuses_more_rows_than_its_working_array():
    lib = _lib()
    most = lib.tuff_argmax_noalloc_max_rows()
    logits = torch.zeros(most + 1, 16, device="cuda")
    out = torch.full((most + 1,), -7, dtype=torch.int32, device="cuda")
    rc = _call(lib, logits, out)
    assert rc == -3 and b"more rows" in lib.tuff_argmax_noalloc_message(rc)
    torch.cuda.synchronize()
    assert (out == -7).all()                                 # nothing ran
    assert _call(lib, logits[:most], out) == 0
    torch.cuda.synchronize()
    assert (out[:most] == 0).all()
