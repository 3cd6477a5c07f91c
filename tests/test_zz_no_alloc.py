"""The allocation-free array sum (emb_array_sum_f32_static) against the ordinary compiled chain.

Some hosts of this library hold device pointers but must not allocate device memory (they live in
another framework's pool, or run where cudaMalloc's synchronisation is not allowed). For them the
library keeps the partial sums, normally a caller-owned scratch buffer, in a fixed device array of
its own. This test calls that entry point through the C ABI twice in a row and checks each result
bit for bit against the chain compiled with --strict and launched through emb_launch with the same
number of blocks (the tolerance the strict reduction tests use: none).
"""

import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def bind(lib):
    lib.emb_array_sum_f32_static.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p]
    return lib


@pytest.mark.parametrize("n,blocks", [(1 << 20, 148), (1 << 20, 1), (1 << 21, 2048), (4096, 64)])
def test_static_scratch_sum_matches_the_compiled_chain_twice_in_a_row(tmp_path, n, blocks):
    """One block, the array's last slot (2048 blocks), and more blocks than 1024-element trips (the idle blocks write
    the sum's identity) besides the usual geometry; and the point of the entry point: the call allocates nothing."""
    import torch
    from emmy_ptx import driver, problems, runner
    lib = bind(driver.library())
    p = problems.array_sum(n=n, grid=blocks, block=256, final_block=256, ident="t")
    folder = problems.write(p, tmp_path)
    rng = np.random.default_rng(42)
    out = torch.zeros(1, dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    for trial in range(2):  # the second call finds the first call's partials in the array
        x = rng.uniform(-1, 1, n).astype(np.float32) * np.float32(trial + 1)
        want = runner.Problem(folder, "strict", inputs={"x": x}).run()["sum_1"]
        xd = torch.from_numpy(x).cuda()
        out.fill_(float("nan"))
        torch.cuda.synchronize()
        if trial == 1:  # (the first call on a device loads the kernels and looks the array's address up)
            free_before, held_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        code = lib.emb_array_sum_f32_static(xd.data_ptr(), n, blocks, out.data_ptr(), ctypes.c_void_p(stream))
        assert code == 0, lib.emb_last_error()
        torch.cuda.synchronize()
        if trial == 1:
            assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_allocated() == held_before
        got = out.cpu().numpy()
        assert got.view(np.uint32)[0] == want.reshape(-1).view(np.uint32)[0], (trial, got, want)


def test_static_scratch_sum_refuses_what_does_not_fit():
    import torch
    from emmy_ptx import driver
    lib = bind(driver.library())
    x = torch.zeros(4096 + 4, device="cuda")
    out = torch.zeros(1, device="cuda")
    assert lib.emb_array_sum_f32_static(x.data_ptr(), 4096, 2049, out.data_ptr(), None) == -2
    assert b"at most 2048 partials" in lib.emb_last_error()
    assert lib.emb_array_sum_f32_static(x.data_ptr(), 4094, 8, out.data_ptr(), None) == -2
    assert lib.emb_array_sum_f32_static(None, 4096, 8, out.data_ptr(), None) == -2
    assert lib.emb_array_sum_f32_static(x.data_ptr() + 4, 4096, 8, out.data_ptr(), None) == -2  # x not on a 16-byte boundary
    assert b"16-byte aligned" in lib.emb_last_error()
