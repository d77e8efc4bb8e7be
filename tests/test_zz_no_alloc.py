"""The allocation-free grid set-up gives exactly what the allocating one gives.

nb_grid_setup_noalloc exists for host programs that are not allowed to call cudaMalloc where they configure a
grid (a plug-in living inside another application's memory budget, a loop that cannot take cudaMalloc's
device-wide synchronisation).  It keeps its scratch in a static device array that all calls share, so this
test calls it twice in a row with different geometries and checks both results against nb_grid_setup, bit for
bit: stale values from the first call must not leak into the second.  The file name sorts last so that a run
stopping at the first failure has already run everything else; the test also passes alone in a fresh process
(the first call on a device does the one-time address look-up)."""
import ctypes

import pytest

pytestmark = pytest.mark.gpu


def _both(nb, L, T, base, growth):
    lib = nb.load()
    a, b = nb.GridDesc(), nb.GridDesc()
    nb.check(lib.nb_grid_setup(ctypes.byref(a), L, T, base, growth, nb.stream_ptr()), "nb_grid_setup")
    nb.check(lib.nb_grid_setup_noalloc(ctypes.byref(b), L, T, base, growth, nb.stream_ptr()), "nb_grid_setup_noalloc")
    return a, b


def test_noalloc_grid_setup_matches_allocating_setup_twice_in_a_row(cuda, nb):
    for (L, T, base, growth) in [(16, 1 << 19, 16, 1.447), (8, 1 << 14, 4, 1.3819)]:
        a, b = _both(nb, L, T, base, growth)
        assert (b.num_levels, b.table_size, b.base_resolution, b.dense_level_start) == \
               (a.num_levels, a.table_size, a.base_resolution, a.dense_level_start)
        assert list(b.scales) == list(a.scales)          # same kernel, same expression: identical bits
        assert list(b.scatter_scales) == list(a.scatter_scales)
        assert all(s > 0 for s in list(b.scales)[:L]) and all(s == 0 for s in list(b.scales)[L:])


def test_noalloc_grid_setup_rejects_sizes_beyond_its_static_scratch(cuda, nb):
    d = nb.GridDesc()
    rc = nb.load().nb_grid_setup_noalloc(ctypes.byref(d), 18, 1 << 14, 16, 1.5, nb.stream_ptr())
    assert rc == 4                                       # NB_ERR_LIMIT
    assert b"16 levels" in nb.load().nb_last_error()
