"""libemmyb200.so loads without a GPU and exports every symbol include/emmy_b200.h declares."""

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as g
    return ctypes.CDLL(str(g.build_library()))


def declared_functions():
    text = (ROOT / "include" / "emmy_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(emb_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_functions()
    assert "emb_launch" in names and "emb_tensor_map" in names and len(names) >= 10
    for n in names:
        assert hasattr(lib, n), n


def test_calls_fail_loudly_without_a_driver_or_with_bad_arguments(lib):
    lib.emb_last_error.restype = ctypes.c_char_p
    assert lib.emb_abi_version() == 2
    code = lib.emb_init(0)
    if code == -1:  # this machine has no CUDA driver: every call says so instead of computing anything
        assert b"libcuda" in lib.emb_last_error()
        assert lib.emb_launch(None, None) == -1
    else:
        assert lib.emb_launch(None, None) == -2 and b"null" in lib.emb_last_error()


def test_product_path_refuses_to_run_without_a_gpu(tmp_path):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from emmy_ptx import driver, problems, runner
    folder = problems.write(problems.array_sum(n=4096, grid=4, block=128, final_block=64, ident="t"), tmp_path)
    with pytest.raises(driver.EmbError):
        runner.Problem(folder)


def test_exchange_record_of_the_header_is_what_the_host_packs(tmp_path):
    """emb_peer_exchange_t (C, include/emmy_b200.h), emb::PeerExchange (the kernels' view) and multi.exchange_record
    (the bytes the host writes) describe the same 88 bytes."""
    import subprocess

    from emmy_ptx import multi
    src = tmp_path / "layout.cpp"
    src.write_text('''
#include <cstddef>
#include <cstdio>
#include "emmy_b200.h"
#include "emb_peer.cuh"
int main() {
    std::printf("%zu %zu %zu %zu %zu %zu\\n", sizeof(emb_peer_exchange_t), offsetof(emb_peer_exchange_t, rank),
                offsetof(emb_peer_exchange_t, step), offsetof(emb_peer_exchange_t, status),
                offsetof(emb_peer_exchange_t, wait_limit_us), sizeof(emb::PeerExchange));
    return !(offsetof(emb::PeerExchange, status) == offsetof(emb_peer_exchange_t, status) &&
             offsetof(emb::PeerExchange, wait_limit_us) == offsetof(emb_peer_exchange_t, wait_limit_us));
}
''')
    exe = tmp_path / "layout"
    templates = ROOT / "emmy-ptx-compiler_b200" / "csrc" / "templates"
    subprocess.run(["nvcc", "-x", "cu", "-I", str(ROOT / "include"), "-I", str(templates), "-o", str(exe), str(src)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()
    assert [int(v) for v in out] == [multi.RECORD_BYTES, 64, 72, 76, 80, multi.RECORD_BYTES]


def test_a_status_word_becomes_an_error_with_code_cta_and_step():
    """What the host makes of a template's bounded wait that gave up (no GPU needed: the word is synthetic)."""
    import pytest

    from emmy_ptx import driver, runner
    runner.raise_on_status("k_matmul", [0, 7, 9, 0, 0, 0, 0, 0])  # nothing happened
    with pytest.raises(driver.EmbError) as err:
        runner.raise_on_status("k_matmul", [3, 41, 1005, 0, 0, 0, 0, 0])
    assert err.value.code == -3
    text = str(err.value)
    assert "k_matmul" in text and "accumulator never completed" in text and "code 3, CTA 41, step 1005" in text
    with pytest.raises(driver.EmbError, match="code 5, CTA 2, step 100"):
        runner.raise_on_status("k_attention", [5, 2, 100])
