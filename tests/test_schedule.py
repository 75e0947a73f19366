"""The integer arithmetic that divides the last round of a persistent grid along K (gpurs_b200/csrc/kernels/
gemm_schedule.hpp), shared by the host and the kernels: compiled here as plain C++ and checked for the properties the
kernels rely on."""
import ctypes as C
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER_DIR = ROOT / "gpurs_b200" / "csrc" / "kernels"

SOURCE = r"""
#include "gemm_schedule.hpp"
extern "C" {
static gemm::StreamSchedule forced(int tiles, int k_blocks, int clusters) {
    return gemm::make_stream_schedule(tiles, k_blocks, clusters, gemm::stream_split_tiles(tiles, k_blocks, clusters, true));
}
int policy_split_tiles(int tiles, int k_blocks, int clusters, int force) { return gemm::stream_split_tiles(tiles, k_blocks, clusters, force != 0); }
int schedule_summary(int tiles, int k_blocks, int clusters, int *out) {
    gemm::StreamSchedule s = forced(tiles, k_blocks, clusters);
    out[0] = s.whole_tiles, out[1] = s.split_tiles, out[2] = s.clusters, out[3] = gemm::max_contributors(s);
    return 0;
}
long long schedule_first_unit(int tiles, int k_blocks, int clusters, int c) { return forced(tiles, k_blocks, clusters).first_unit(c); }
int schedule_owner(int tiles, int k_blocks, int clusters, long long unit) { return forced(tiles, k_blocks, clusters).owner(unit); }
int schedule_contributors(int tiles, int k_blocks, int clusters, int r, int *first) {
    gemm::StreamSchedule s = forced(tiles, k_blocks, clusters);
    *first = s.first_contributor(r);
    return s.contributors(r);
}
}
"""


@pytest.fixture(scope="module")
def schedule(tmp_path_factory):
    folder = tmp_path_factory.mktemp("schedule")
    (folder / "schedule.cpp").write_text(SOURCE)
    library = folder / "libschedule.so"
    subprocess.run(["g++", "-std=c++17", "-O2", "-Wall", "-Wextra", "-Werror", "-shared", "-fPIC", "-I", str(HEADER_DIR), str(folder / "schedule.cpp"),
                    "-o", str(library)], check=True)
    lib = C.CDLL(str(library))
    lib.schedule_first_unit.restype = C.c_longlong
    lib.schedule_first_unit.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int]
    lib.schedule_owner.argtypes = [C.c_int, C.c_int, C.c_int, C.c_longlong]
    return lib


def summary(lib, tiles, k_blocks, clusters):
    out = (C.c_int * 4)()
    lib.schedule_summary(tiles, k_blocks, clusters, out)
    return tuple(out)


def test_when_the_last_round_is_split(schedule):
    policy = schedule.policy_split_tiles
    # never: fewer tiles than groups, exact multiples, one-block depths
    for tiles, k_blocks, clusters in [(60, 64, 74), (148, 64, 74), (256, 1, 74)]:
        assert policy(tiles, k_blocks, clusters, 0) == 0 and policy(tiles, k_blocks, clusters, 1) == 0
    # only when forced: the idle share of the last round is worth less than about 30 K-blocks
    for tiles, k_blocks, clusters in [(1024, 128, 74), (128, 64, 74), (74 * 3 + 60, 64, 74), (10, 8, 4)]:
        assert policy(tiles, k_blocks, clusters, 0) == 0 and policy(tiles, k_blocks, clusters, 1) == tiles % clusters
    # the reference example on CTA pairs: 256 tiles on 74 groups = 3 whole rounds + 34 tiles over all 74 groups
    assert policy(256, 64, 74, 0) == 34 and summary(schedule, 256, 64, 74)[:3] == (222, 34, 74)
    # FP8 4096 x 7168 x 7168: 448 tiles, 4 left over: at most 4 groups per tile take part
    assert policy(448, 56, 74, 0) == 4 and summary(schedule, 448, 56, 74)[:3] == (444, 4, 16)


@pytest.mark.parametrize("tiles,k_blocks,clusters", [(256, 64, 74), (448, 56, 74), (10, 2, 4), (15, 16, 6), (24, 18, 7), (9, 3, 8), (512, 64, 148),
                                                      (75, 7, 74), (300, 1000, 148), (149, 2, 148)])
def test_shares_tile_the_units_and_contributors_are_consistent(schedule, tiles, k_blocks, clusters):
    whole, split, groups, most = summary(schedule, tiles, k_blocks, clusters)
    if split == 0:
        pytest.skip("no split round for this shape")
    assert whole % clusters == 0 and whole + split == tiles and groups <= clusters
    units = split * k_blocks
    firsts = [schedule.schedule_first_unit(tiles, k_blocks, clusters, c) for c in range(groups + 1)]
    assert firsts[0] == 0 and firsts[-1] == units and all(a <= b for a, b in zip(firsts, firsts[1:]))
    # every unit belongs to exactly the group whose share holds it
    for unit in range(units):
        owner = schedule.schedule_owner(tiles, k_blocks, clusters, unit)
        assert firsts[owner] <= unit < firsts[owner + 1]
    # contributors of a tile = the groups whose shares meet its K-blocks, numbered from the first
    seen_most = 0
    for r in range(split):
        first = C.c_int()
        count = schedule.schedule_contributors(tiles, k_blocks, clusters, r, C.byref(first))
        holders = sorted({schedule.schedule_owner(tiles, k_blocks, clusters, unit) for unit in range(r * k_blocks, (r + 1) * k_blocks)})
        assert holders == list(range(first.value, first.value + count))
        seen_most = max(seen_most, count)
    assert seen_most == most
    # shares differ by at most one unit: nobody works through a whole extra tile's depth
    sizes = [b - a for a, b in zip(firsts, firsts[1:])]
    assert max(sizes) - min(sizes) <= 1


def test_sweep_of_small_grids(schedule):
    """Every (tiles, depth, groups) of a small sweep: no group that takes part has an empty share, and every split tile's
    K-blocks are held by a contiguous range of groups that matches what the kernels will count."""
    checked = 0
    for clusters in list(range(1, 13)) + [37, 74, 148]:
        for tiles in list(range(1, 3 * clusters + 2)) if clusters <= 12 else [clusters + 1, clusters + 5, 2 * clusters + clusters // 2, 3 * clusters + 7]:
            for k_blocks in (1, 2, 3, 5, 8, 31, 64):
                whole, split, groups, most = summary(schedule, tiles, k_blocks, clusters)
                assert whole + split == tiles
                if split == 0:
                    continue
                checked += 1
                units = split * k_blocks
                firsts = [schedule.schedule_first_unit(tiles, k_blocks, clusters, c) for c in range(groups + 1)]
                assert firsts[0] == 0 and firsts[-1] == units
                assert all(b > a for a, b in zip(firsts, firsts[1:])), (tiles, k_blocks, clusters)     # no empty share
                for r in range(split):
                    first = C.c_int()
                    count = schedule.schedule_contributors(tiles, k_blocks, clusters, r, C.byref(first))
                    low, high = r * k_blocks, (r + 1) * k_blocks
                    holders = [c for c in range(groups) if firsts[c] < high and firsts[c + 1] > low]
                    assert holders == list(range(first.value, first.value + count)), (tiles, k_blocks, clusters, r)
                    assert count <= most
    assert checked > 200
