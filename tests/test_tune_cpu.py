"""Measured selection, the host half (no GPU): the duel protocol with a fake timer and the verdict file.

The reference's rules (jit/gpu/tier/split.go:18-75): candidates in order, a dispersed sample (IQR / median above
0.10) is refused rather than rounded, a later candidate must beat the best so far by more than 1 %, nothing usable
means the table's answer stands; verdicts persist keyed by device + driver + build and a damaged entry is no
entry (jit/gpu/tier/choose.go:196-216)."""
import ctypes as C

from jitllm_b200 import _lib


def _duel(table, gate=0.10, margin=0.01):
    """table[c] = the rates candidate c's timed rounds return (a value <= 0 = the run failed)."""
    L = _lib.load()
    calls = []

    def timer(_user, cand, rnd):
        calls.append((cand, rnd))
        return float(table[cand][rnd])
    cb = _lib.TUNE_TIMER(timer)
    n, rounds = len(table), len(table[0])
    refused = (C.c_int * n)()
    med = (C.c_double * n)()
    w = L.jl_tune_duel(n, rounds, cb, None, gate, margin, refused, med)
    return w, list(refused), list(med), calls


def test_the_table_pick_wins_a_tie_and_a_clear_challenger_wins():
    flat = [100.0] * 9
    w, refused, med, calls = _duel([flat, [100.9] * 9, [100.5] * 9])
    assert w == 0 and refused == [0, 0, 0] and med[1] == 100.9       # within 1 %: the trial cannot tell them apart
    assert calls[:9] == [(0, r) for r in range(9)] and len(calls) == 27
    w, _, _, _ = _duel([flat, [101.5] * 9, [102.0] * 9])
    assert w == 1                                                    # 102.0 does not beat 101.5 by 1 %
    w, _, _, _ = _duel([flat, [101.5] * 9, [103.0] * 9])
    assert w == 2


def test_a_dispersed_sample_is_refused_not_rounded():
    noisy = [100.0, 300.0, 150.0, 250.0, 120.0, 280.0, 200.0, 90.0, 310.0]   # median 200, IQR 160: far above 0.10
    steady = [100.0, 100.5, 99.5, 100.2, 99.8, 100.1, 99.9, 100.3, 99.7]
    w, refused, med, _ = _duel([steady, noisy])
    assert w == 0 and refused == [0, 1] and med[1] == 0.0
    # the table's own pick dispersed: a steady challenger takes it even when slower
    w, refused, _, _ = _duel([noisy, [50.0] * 9])
    assert w == 1 and refused == [1, 0]
    # nothing usable: no verdict
    w, refused, _, _ = _duel([noisy, noisy])
    assert w == -1 and refused == [1, 1]


def test_a_failed_run_refuses_the_candidate_and_stops_timing_it():
    bad = [100.0, 0.0] + [100.0] * 7
    w, refused, _, calls = _duel([[90.0] * 9, bad, [95.0] * 9])
    assert w == 2 and refused == [0, 1, 0]
    assert [c for c in calls if c[0] == 1] == [(1, 0), (1, 1)]


def test_median_and_quartiles_are_of_the_sorted_sample():
    # 9 rounds: median = 5th smallest, IQR = 7th - 3rd smallest
    s = [10, 50, 11, 12, 13, 14, 15, 16, 9]                          # sorted: 9 10 11 12 13 14 15 16 50
    w, refused, med, _ = _duel([[float(v) for v in s]], gate=0.31)
    assert w == 0 and med[0] == 13.0 and refused == [0]              # (15 - 11) / 13 = 0.307
    w, refused, _, _ = _duel([[float(v) for v in s]], gate=0.30)
    assert w == -1 and refused == [1]


def test_the_verdict_file_round_trips_and_a_damaged_entry_is_no_entry(tmp_path):
    L = _lib.load()
    d = str(tmp_path / "cache").encode()
    buf = C.create_string_buffer(64)
    assert L.jl_tune_cache_lookup(d, b"k1", buf, 64) == 0            # no directory yet
    assert L.jl_tune_cache_save(d, b"dev0/12-4096x4096x1", b"3 16 2 1 4") == 1
    assert L.jl_tune_cache_save(d, b"dev0/12-14336x4096x1", b"1 4 4 4 1") == 1
    assert L.jl_tune_cache_lookup(d, b"dev0/12-4096x4096x1", buf, 64) == 1 and buf.value == b"3 16 2 1 4"
    assert L.jl_tune_cache_lookup(d, b"dev0/12-4096x4096", buf, 64) == 0      # a prefix of a key is not the key
    assert L.jl_tune_cache_lookup(d, b"dev1/12-4096x4096x1", buf, 64) == 0    # another device / driver / build
    assert L.jl_tune_cache_save(d, b"dev0/12-4096x4096x1", b"1 8 2 2 1") == 1   # overwritten, not appended
    assert L.jl_tune_cache_lookup(d, b"dev0/12-4096x4096x1", buf, 64) == 1 and buf.value == b"1 8 2 2 1"
    text = (tmp_path / "cache" / "jl_select1").read_text()
    assert text.count("dev0/12-4096x4096x1") == 1 and text.count("\n") == 2
    # a torn last line (no newline) is not an entry; the next save drops it
    with open(tmp_path / "cache" / "jl_select1", "a") as f:
        f.write("dev0/12-1024x4096x1 3 16")
    assert L.jl_tune_cache_lookup(d, b"dev0/12-1024x4096x1", buf, 64) == 0
    assert L.jl_tune_cache_save(d, b"dev0/12-512x512x1", b"2 16 1 1 1") == 1
    assert "dev0/12-1024x4096x1" not in (tmp_path / "cache" / "jl_select1").read_text()
    # keys and values that would break the line format are refused
    assert L.jl_tune_cache_save(d, b"a b", b"1") == 0 and L.jl_tune_cache_save(d, b"a", b"1\n2") == 0
    assert L.jl_tune_cache_save(b"", b"a", b"1") == 0


def test_the_device_key_changes_with_uuid_driver_and_build():
    L = _lib.load()

    def key(uuid, drv, build):
        out = C.create_string_buffer(17)
        L.jl_tune_device_key(uuid, drv, build, out)
        return out.value
    u0, u1 = bytes(range(16)), bytes(range(1, 17))
    base = key(u0, 12090, b"abc")
    assert len(base) == 16 and base == key(u0, 12090, b"abc")
    assert len({base, key(u1, 12090, b"abc"), key(u0, 12080, b"abc"), key(u0, 12090, b"abd")}) == 4
    assert len(L.jl_build_id()) == 16                               # the in-tree build stamps a source hash
