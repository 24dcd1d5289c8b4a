"""The page and slot index arithmetic that the kernels share (tuff_b200/csrc/index.cuh), run on
the host: the header compiles without CUDA, and this test calls it through a small C++ file."""
import ctypes
import os
import shutil
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib(tmp_path_factory):
    cxx = shutil.which("g++") or shutil.which("c++")
    assert cxx, "a C++ compiler is needed for the host build of the index helpers"
    out = str(tmp_path_factory.mktemp("index") / "index_host.so")
    subprocess.run([cxx, "-O1", "-std=c++17", "-shared", "-fPIC", "-I", os.path.join(ROOT, "tuff_b200", "csrc"),
                    "-x", "c++", os.path.join(ROOT, "tests", "index_host.cpp"), "-o", out], check=True)
    h = ctypes.CDLL(out)
    h.h_page_elem.restype = ctypes.c_ulonglong
    h.h_page_elem.argtypes = [ctypes.c_longlong] + [ctypes.c_int] * 5
    h.h_slot_elem.restype = ctypes.c_ulonglong
    h.h_slot_elem.argtypes = [ctypes.c_longlong, ctypes.c_ulonglong]
    for f in (h.h_page_ok, h.h_slot_ok, h.h_row_ok):
        f.argtypes = [ctypes.c_longlong, ctypes.c_longlong]
    return h


def test_a_position_finds_its_page_entry_and_offset(lib):
    rng = np.random.default_rng(0)
    for page_size in (1, 2, 4, 16, 64, 100):
        for pos in [0, 1, page_size - 1, page_size, page_size + 1, 8191, 131071] + rng.integers(0, 1 << 20, 20).tolist():
            e, o = lib.h_page_entry(pos, page_size), lib.h_page_offset(pos, page_size)
            assert 0 <= o < page_size and e * page_size + o == pos


def test_elements_of_pages_and_slots_do_not_overlap_and_do_not_wrap(lib):
    G, page, hd = 3, 8, 48
    seen = set()
    for p in range(4):
        for g in range(G):
            for o in range(page):
                first = lib.h_page_elem(p, g, o, G, page, hd)
                assert first % hd == 0 and first not in seen
                seen.add(first)
    assert seen == {i * hd for i in range(4 * G * page)}                   # dense: [page][kv_head][offset][hd]
    # a pool of 180 GB: indices beyond 32 bits stay exact
    assert lib.h_page_elem(3_000_000, 7, 63, 8, 64, 128) == ((3_000_000 * 8 + 7) * 64 + 63) * 128
    assert lib.h_slot_elem(70_000, 3 * 65_536) == 70_000 * 3 * 65_536


def test_range_checks_take_the_ends_and_refuse_one_beyond(lib):
    for ok, n in ((lib.h_page_ok, 17), (lib.h_slot_ok, 5), (lib.h_row_ok, 1)):
        assert ok(0, n) and ok(n - 1, n)
        assert not ok(-1, n) and not ok(n, n) and not ok(1 << 40, n) and not ok(0, 0)
    # a table of 4 entries with pages of 16 holds positions 0..63
    assert lib.h_page_entry_ok(0, 16, 4) and lib.h_page_entry_ok(63, 16, 4)
    assert not lib.h_page_entry_ok(64, 16, 4) and not lib.h_page_entry_ok(-1, 16, 4)
