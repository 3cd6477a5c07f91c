"""The cluster-sharing plan: the shape it gives the reference's column-recomputing MLP, and its refusals."""

import json
from pathlib import Path

import pytest

from emmy_ptx import clusterize, ir, problems


@pytest.fixture(scope="module")
def tile():
    here = Path(__file__).parent / "golden"
    case = next(c for c in json.loads((here / "oracle_cases.json").read_text()) if c["name"] == "ex_k_gelu_mlp")
    return ir.parse(case["body"][0])


def test_plan_shape_for_the_shipped_example(tile):
    p = clusterize.plan(tile, 4096, 8)
    assert isinstance(p, clusterize.ClusterPlan)
    assert p.trips == 64 and p.slots == 8 and p.step == 8 and p.values == ("v5",)
    assert [ir.kind(s) for s in p.shared] == ["Loop"] + ["Assign"] * 5  # the dot product and the erf-GELU
    assert [ir.kind(s) for s in p.own] == ["Load", "Assign", "Accum"]  # w2[unit, column], product, fold
    assert [ir.kind(s) for s in p.after] == ["WarpShuffle", "Cond"]


def test_refusals(tile):
    assert "threads outside the Tile" in clusterize.plan(tile, 4100, 8)
    assert isinstance(clusterize.plan(tile, 4096, 8), clusterize.ClusterPlan)
    # a block of 16 threads holds two columns of the 128: the column coordinate is neither inside a block nor across whole blocks
    assert "straddles" in clusterize.plan(tile, 2048, 16)
    # a loop that is not pure (a Write inside) is left alone
    loop = next(s for s in tile.body if ir.kind(s) == "StridedLoop")
    w = ir.Write(output="matmul_1", index=(ir.Var(name="a0"), ir.Var(name="a1")), values=("v5",))
    dirty = tile.replace(body=tuple(s.replace(body=s.body + (w,)) if s is loop else s for s in tile.body))
    assert "not pure" in clusterize.plan(dirty, 4096, 8)
    # too little shared work
    small = loop.replace(body=(loop.body[0].replace(axis=ir.Axis(name="a3", extent=2)),) + loop.body[1:])
    tiny = tile.replace(body=tuple(small if s is loop else s for s in tile.body))
    assert "shared inner iterations" in clusterize.plan(tiny, 4096, 8)
    # a trip count that does not divide among 8 blocks
    odd = loop.replace(axis=ir.Axis(name="a2", extent=8 * 63))
    assert "trip count" in clusterize.plan(tile.replace(body=tuple(odd if s is loop else s for s in tile.body)), 4096, 8)


def test_the_workload_mlp_is_not_clustered_by_this_rule():
    """Its blocks hold 32 (column, lane) groups each, so no coordinate steps one block at a time: the tensor-core
    template serves it instead."""
    p = problems.gelu_mlp(tokens=8, d_model=64, hidden=64, lanes=8, block=64)
    t = p["kernels"][0]["body"][0]
    assert isinstance(clusterize.plan(t, p["kernels"][0]["grid"], 64), str)
