"""The four fp8 conversions (from_f8e4m3, from_f8e5m2, to_f8e4m3, to_f8e5m2): all 256 codes of each format decoded, and
float32 values of every kind encoded - ties, the largest finite values, saturation, subnormals, infinities, NaN - as the
reference's test does (tests/test_gpu_lowering.py:554-599). That test compares with emmy's own tables, which are not
available; what pins the answers here is the reference's prose definition (emmy_ptx/elementwise.py:100-123,
docs/DESIGN.md:619-628: value = byte code, exact widening, round to nearest even, saturate to the largest finite value,
NaN to 0x7f) spelled out as explicit expectations below, and ml_dtypes for the bulk."""

import ml_dtypes
import numpy as np
import pytest

from emmy_ptx import runner
from emmy_ptx.frontend import Buffer, KernelSource, Launch
from emmy_ptx.ir import Assign, Axis, BinaryExpr, Cond, Literal, Load, Tile, Var, Write, datatype
from oracle import ir_oracle

N = 1024
FORMATS = {"f8e4m3": (ml_dtypes.float8_e4m3fn, 448.0), "f8e5m2": (ml_dtypes.float8_e5m2, 57344.0)}
SPECIAL = [0.0, -0.0, 448.0, 464.0, 480.0, -500.0, 57344.0, 61440.0, 1e30, -1e30, np.inf, -np.inf, np.nan, 2.0 ** -9, 2.0 ** -10,
           2.0 ** -17]
# the byte codes the definition gives the special values
EXPECTED = {"f8e4m3": [0x00, 0x80, 0x7E, 0x7E, 0x7E, 0xFE, 0x7E, 0x7E, 0x7E, 0xFE, 0x7E, 0xFE, 0x7F, 0x01, 0x00, 0x00],
            # e5m2: 448 = 1.75 * 2^8 is 0x5F; 464 rounds down to it; 480 ties between 448 (odd mantissa) and 512 = 0x60 (even);
            # -500 is nearer -512; 61440 ties up to 65536, which is past the largest finite value 57344 = 0x7B; 2^-9 and 2^-10
            # are normal (exponent fields 6 and 5); 2^-17 is half the smallest subnormal and ties to zero
            "f8e5m2": [0x00, 0x80, 0x5F, 0x5F, 0x60, 0xE0, 0x7B, 0x7B, 0x7B, 0xFB, 0x7B, 0xFB, 0x7F, 0x18, 0x14, 0x00]}


def values():
    rng = np.random.default_rng(3)
    return np.concatenate([rng.standard_normal(N // 2) * 100, rng.standard_normal(N // 4) * 0.01,
                           np.ldexp(rng.integers(8, 32, N // 4 - 16), -rng.integers(0, 24, N // 4 - 16)), SPECIAL]).astype(np.float32)


def kernel(fmt: str):
    i = Var(name="i")
    return (Tile(axes=(Axis(name="i", extent=N),), body=(
        Load(names=("x",), input="xs", index=(i,), dtype=None),
        Assign(name="c", op=f"to_{fmt}", args=("x",), dtype=datatype(fmt)),
        Write(output="enc", index=(i,), values=("c",), value_dtype=None),
        Cond(cond=BinaryExpr(op="<", left=i, right=Literal(value=256, dtype="int")), body=(
            Load(names=("k",), input="codes", index=(i,), dtype=None),
            Assign(name="v", op=f"from_{fmt}", args=("k",), dtype=datatype("f32")),
            Write(output="dec", index=(i,), values=("v",), value_dtype=None)), else_body=())),
        block_threads=256, aux_threads=0, raster_axes=None, raster_group=None, raster_orient="m"),)


def buffers(fmt: str):
    return {"xs": Buffer("xs", (N,), "f32"), "codes": Buffer("codes", (256,), fmt), "enc": Buffer("enc", (N,), fmt),
            "dec": Buffer("dec", (256,), "f32")}


def arrays():
    return {"xs": values(), "codes": np.arange(256, dtype=np.uint8), "enc": np.zeros(N, np.uint8), "dec": np.zeros(256, np.float32)}


@pytest.mark.parametrize("fmt", sorted(FORMATS))
def test_the_oracle_follows_the_definition(fmt):
    np_type, largest = FORMATS[fmt]
    bufs = arrays()
    ir_oracle.run(kernel(fmt), bufs, N // 256, 256)
    assert bufs["enc"][-len(SPECIAL):].tolist() == EXPECTED[fmt]
    want = np.arange(256, dtype=np.uint8).view(np_type).astype(np.float32)
    assert np.array_equal(bufs["dec"], want, equal_nan=True)
    # every encoded value decodes to the nearest representable one (ties aside, which the explicit cases cover)
    x = bufs["xs"][:-len(SPECIAL)]
    back = bufs["enc"][:-len(SPECIAL)].view(np_type).astype(np.float32)
    finite = np.sort(want[np.isfinite(want)])
    nearest = finite[np.abs(finite[None, :] - np.clip(x, -largest, largest)[:, None]).argmin(axis=1)]
    assert np.array_equal(np.abs(back - x) <= np.abs(nearest - x) + 0, np.ones(x.size, bool))


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["optimized", "strict"])
@pytest.mark.parametrize("fmt", sorted(FORMATS))
def test_the_gpu_agrees_with_the_oracle_on_every_code_and_kind_of_value(fmt, mode):
    src = KernelSource("k_fp8", kernel(fmt), ("xs", "codes", "enc", "dec"), buffers(fmt), Launch(N // 256, 256, 0), frozenset({"enc", "dec"}))
    got = runner.run_source(src, arrays(), mode)
    want = arrays()
    ir_oracle.run(kernel(fmt), want, N // 256, 256)
    assert np.array_equal(got["enc"], want["enc"])
    assert np.array_equal(got["dec"], want["dec"], equal_nan=True)
