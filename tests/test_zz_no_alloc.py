"""The sampling entry point that allocates nothing (csrc/kernels/sampling_no_alloc.h), called
through its exported C symbol, against the regular entry point.

Some programs that embed these kernels cannot allocate device memory when they sample: they have
given all free GPU memory to their own pools, or they run a loop that must not enter the CUDA
allocator. For them `llm_sample_no_alloc` keeps its scratch in a fixed array inside the library.
This test loads the library with ctypes, as such a program would, calls the symbol twice in a row
(the array is shared between calls and keeps the last call's contents) and expects exactly the
tokens of `llm_sample`, whose scratch the caller provides. It also checks that a request larger
than the built-in scratch is refused with a message rather than run.

The file name sorts last so that a run that stops at the first failure has already run every other
test; the test does not depend on them and passes alone in a fresh process as well.
"""
import ctypes
from ctypes import c_int, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
MAX_ROWS = 256  # LLM_SAMPLE_NO_ALLOC_MAX_ROWS


def _lib():
    from llmengine.csrc import build
    lib = ctypes.CDLL(build.kernel_library_path("core"))
    lib.llm_last_error.restype = ctypes.c_char_p
    return lib


def _ptr(t):
    return c_void_p(0 if t is None else t.data_ptr())


def _regular(lib, logits, temps, seeds, draws, n, vocab):
    out = torch.full((n,), -1, dtype=torch.int32, device=logits.device)
    chunks = lib.llm_sample_chunks(c_int(vocab))
    scratch = torch.empty(2 * n * chunks, dtype=torch.int32, device=logits.device)
    rc = lib.llm_sample(_ptr(logits), c_longlong(logits.stride(0)), _ptr(temps), _ptr(seeds), _ptr(draws), _ptr(out),
                        c_int(n), c_int(vocab), _ptr(scratch), c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.llm_last_error().decode()
    return out


def _no_alloc(lib, logits, temps, seeds, draws, n, vocab):
    out = torch.full((n,), -1, dtype=torch.int32, device=logits.device)
    rc = lib.llm_sample_no_alloc(_ptr(logits), c_longlong(logits.stride(0)), _ptr(temps), _ptr(seeds), _ptr(draws),
                                 _ptr(out), c_int(n), c_int(vocab), c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, lib.llm_last_error().decode()
    return out


def test_no_alloc_sampling_matches_the_regular_entry_point_twice_in_a_row():
    lib = _lib()
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(123)
    # two calls in a row with different shapes: the second must not see anything of the first
    cases = [(37, 128256, True), (5, 509, False), (MAX_ROWS, 5003, True)]
    for n, vocab, sampled in cases:
        logits = torch.randn(n, vocab, generator=g).to(dev)
        logits[0, vocab // 3] = logits[0, vocab - 1] = 40.0  # a tie: the lower index wins
        temps = seeds = draws = None
        if sampled:
            temps = (torch.rand(n, generator=g) * 1.5).to(dev)
            temps[::3] = 0.0  # greedy rows among sampled ones
            seeds = torch.randint(0, 2 ** 31 - 1, (n,), generator=g, dtype=torch.int32).to(dev)
            draws = torch.randint(0, 1000, (n,), generator=g, dtype=torch.int32).to(dev)
        want = _regular(lib, logits, temps, seeds, draws, n, vocab)
        first = _no_alloc(lib, logits, temps, seeds, draws, n, vocab)
        second = _no_alloc(lib, logits, temps, seeds, draws, n, vocab)
        torch.cuda.synchronize()
        assert torch.equal(first, want) and torch.equal(second, want)
        assert int(want[0]) == vocab // 3 or sampled
        assert int(want.min()) >= 0 and int(want.max()) < vocab


def test_no_alloc_sampling_refuses_more_rows_than_its_scratch_holds():
    lib = _lib()
    dev = torch.device("cuda:0")
    n = MAX_ROWS + 1
    logits = torch.zeros(n, 64, device=dev)
    out = torch.zeros(n, dtype=torch.int32, device=dev)
    rc = lib.llm_sample_no_alloc(_ptr(logits), c_longlong(64), _ptr(None), _ptr(None), _ptr(None), _ptr(out), c_int(n),
                                 c_int(64), c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0 and b"exceed the built-in scratch" in lib.llm_last_error()
    torch.cuda.synchronize()


def test_no_alloc_sampling_at_the_full_extent_of_its_scratch():
    """The largest request the built-in array takes: 256 rows, the vocabulary scanned in 64 chunks
    (any vocabulary above 258,048 entries), so that the last (value, index) words of the array are
    written and read. Greedy rows are checked against an argmax taken by another library on the
    host, not only against the regular entry point, which shares the kernels."""
    lib = _lib()
    dev = torch.device("cuda:0")
    n, vocab = MAX_ROWS, 258048 + 1001
    assert lib.llm_sample_chunks(c_int(vocab)) == 64
    g = torch.Generator(device=dev).manual_seed(7)
    logits = torch.randn(n, vocab, generator=g, device=dev)
    logits[2, vocab - 1] = 50.0      # the winner sits in the last chunk's last place
    logits[4, 0] = logits[4, vocab - 2] = 50.0  # a tie across the first and the last chunk: the lower index wins
    temps = torch.zeros(n, device=dev)
    temps[1::2] = 0.8                # every other row is sampled
    seeds = torch.arange(n, dtype=torch.int32, device=dev)
    draws = torch.full((n,), 5, dtype=torch.int32, device=dev)
    want = _regular(lib, logits, temps, seeds, draws, n, vocab)
    first = _no_alloc(lib, logits, temps, seeds, draws, n, vocab)
    second = _no_alloc(lib, logits, temps, seeds, draws, n, vocab)
    torch.cuda.synchronize()
    assert torch.equal(first, want) and torch.equal(second, want)
    host = logits[0::2].cpu().numpy().argmax(axis=1)  # numpy: the first index of the maximum
    assert first[0::2].cpu().tolist() == host.tolist()
    assert int(first[4]) == 0 and int(first[2]) == vocab - 1
