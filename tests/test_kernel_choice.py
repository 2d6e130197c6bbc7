"""Which tcgen05 kernel a prompt-sized product runs on is decided on the host (`llm_gemm_tc_form` in
gemm_tc.cu) from the sizes alone, so it is checked here without a GPU: the choices for the layer
sizes that were measured on B200, and the rules that hold for every size. CTA pairs are off by
default; the tests of the estimate switch them to "where estimated faster" (-1) first."""
import ctypes

import pytest

from llmengine.csrc.build import kernel_library_path

ONE_TILE, PERSISTENT_256, PERSISTENT_192, PAIRS = range(4)


@pytest.fixture(scope="module")
def lib():
    lib = ctypes.CDLL(kernel_library_path("tensorcore"))  # compiled at the first call; loads without a GPU
    yield lib
    lib.llm_gemm_tc_pair(0)  # the library's default: never
    lib.llm_gemm_tc_persistent(1)


# (tokens, outputs, inputs, SwiGLU epilogue) -> the faster form as measured (2,048-token prompts at the
# q|k|v, o, gate|up and down sizes of the Llama 3.2 1B, 3.2 3B and 3.1 8B layers)
MEASURED = [
    ((2048, 3072, 2048, 0), PERSISTENT_192), ((2048, 2048, 2048, 0), ONE_TILE), ((2048, 16384, 2048, 1), PAIRS),
    ((2048, 2048, 8192, 0), PAIRS), ((2048, 5120, 3072, 0), PERSISTENT_192), ((2048, 16384, 3072, 1), PAIRS),
    ((2048, 3072, 8192, 0), PERSISTENT_192), ((2048, 6144, 4096, 0), PAIRS), ((2048, 4096, 4096, 0), PAIRS),
    ((2048, 28672, 4096, 1), PAIRS), ((2048, 4096, 14336, 0), PAIRS),
]


@pytest.mark.parametrize("shape,form", MEASURED)
def test_measured_shapes_get_the_faster_kernel(lib, shape, form):
    lib.llm_gemm_tc_pair(-1)
    lib.llm_gemm_tc_persistent(1)
    assert lib.llm_gemm_tc_form(*shape) == form


def test_rules_of_the_choice(lib):
    lib.llm_gemm_tc_pair(-1)
    lib.llm_gemm_tc_persistent(1)
    for m in (65, 100, 128, 129, 300, 2048, 8192):
        for n in (16, 200, 256, 3000, 16384, 128256):
            for k in (64, 2048, 14336):
                for swiglu in (0, 1):
                    if swiglu and n % 256:
                        continue
                    f = lib.llm_gemm_tc_form(m, n, k, swiglu)
                    if m <= 128 or n < 256:
                        assert f != PAIRS  # a pair needs two tiles of 128 tokens and 256 outputs
                    if n < 256:
                        assert f == ONE_TILE
                    if swiglu:
                        assert f != PERSISTENT_192  # gate and up rows come in blocks of 256
                    if f in (PERSISTENT_256, PERSISTENT_192):
                        tiles = -(-m // 128) * -(-n // (256 if f == PERSISTENT_256 else 192))
                        assert tiles > 148  # persistent only where some SM gets a second tile
    # short products of one round never go to pairs (their later start is not earned back)
    assert lib.llm_gemm_tc_form(2048, 2048, 2048, 0) != PAIRS and lib.llm_gemm_tc_form(256, 256, 64, 0) != PAIRS


def test_switches(lib):
    shape = (2048, 16384, 2048, 1)
    lib.llm_gemm_tc_pair(0)
    assert lib.llm_gemm_tc_form(*shape) == PERSISTENT_256
    lib.llm_gemm_tc_persistent(0)
    assert lib.llm_gemm_tc_form(*shape) == ONE_TILE
    lib.llm_gemm_tc_pair(1)
    assert lib.llm_gemm_tc_form(*shape) == PAIRS and lib.llm_gemm_tc_form(256, 256, 64, 0) == PAIRS
    assert lib.llm_gemm_tc_form(128, 4096, 4096, 0) != PAIRS  # one tile of tokens: nothing to pair
    lib.llm_gemm_tc_pair(0)
    lib.llm_gemm_tc_persistent(1)
