"""Launch shapes of the device path, checked on the CPU: for every collective plan, message
size, rank count, window size and grid limit, each CTA's slots must lie inside its staging
buffer, the steps must cover the message and the epochs must match what the kernels consume.
The same check runs before every real launch (src/device/planner.h: check_geometry)."""
import ctypes as C

import pytest

from hxccl_b200 import _lib as L

KINDS = {"xchg": 0, "sliced": 1, "roles": 2, "ring": 3, "ring_rs": 4}


def plan(kind, amount, n, half, max_ctas=0, knob=None, value=0):
    lib = L.lib()
    lib.hxcclTestPlan.argtypes = [C.c_int, C.c_size_t, C.c_int, C.c_size_t, C.c_int, C.c_char_p, C.c_long,
                                  C.POINTER(C.c_size_t), C.c_char_p, C.c_size_t]
    shape = (C.c_size_t * 5)()
    why = C.create_string_buffer(256)
    rc = lib.hxcclTestPlan(KINDS[kind], amount, n, half, max_ctas, knob.encode() if knob else None, value, shape, why, 256)
    return rc, list(shape), why.value.decode()


SIZES = [1, 15, 16, 17, 4099, 65536, 262144, 262145, (1 << 20) + 16, 3 << 20, (64 << 20) + 48, 256 << 20, 1 << 30, (1 << 30) + 4]


@pytest.mark.parametrize("kind", list(KINDS))
def test_every_plan_fits_its_window(kind):
    bad = []
    for n in (1, 2, 3, 4, 8, 16):
        if kind in ("ring", "ring_rs") and n < 2:
            continue
        for half in (3 << 20, 61 << 20, 253 << 20):
            for max_ctas in (0, 1, 8, 48, 512):
                for amount in SIZES:
                    rc, shape, why = plan(kind, amount, n, half, max_ctas)
                    if rc != 0:
                        bad.append((n, half, max_ctas, amount, shape, why))
    assert not bad, bad[:5]


def test_knobs_keep_plans_inside_the_window():
    for knob, values in (("sub_max", (16, 4096, 1 << 20)), ("single_sub_max", (16, 1 << 22)), ("min_steps", (2, 64)),
                         ("roles_sub", (16, 4096, 1 << 22)), ("ring_sub", (16, 4096, 1 << 22)), ("threads", (256, 512))):
        for v in values:
            for kind in KINDS:
                for n in (2, 8):
                    for amount in (4099, 3 << 20, 256 << 20):
                        rc, shape, why = plan(kind, amount, n, 61 << 20, 0, knob, v)
                        assert rc == 0, (knob, v, kind, n, amount, shape, why)


def test_shapes_of_the_measured_defaults():
    # 256 MiB on two ranks: the ring runs 128 CTAs in two rounds of 512 KiB hops
    rc, (ctas, threads, steps, epochs, sub), _ = plan("ring", 128 << 20, 2, 253 << 20)
    assert rc == 0 and (ctas, threads, steps, epochs, sub) == (128, 512, 2, 2 * 2 + 2, 512 << 10)
    # 256 MiB two-shot on four ranks: pipelined steps of at most 128 KiB per CTA and slice (a quarter
    # of the staging area holds a little less than four ranks x 128 CTAs x 128 KiB x two phases)
    rc, (ctas, threads, steps, epochs, sub), _ = plan("sliced", 256 << 20, 4, 253 << 20)
    assert rc == 0 and ctas == 128 and steps == 5 and epochs == 7 and sub == (512 << 10) // 5 // 16 * 16 + 16
    # 64 MiB on eight ranks fits one step
    rc, (ctas, threads, steps, epochs, sub), _ = plan("sliced", 64 << 20, 8, 253 << 20)
    assert rc == 0 and (steps, epochs, sub) == (1, 1, 64 << 10)
    assert plan("ring", 1024, 1, 1 << 20)[0] == L.INVALID_ARGUMENT


def test_tune_file(tmp_path, monkeypatch):
    good = tmp_path / "tune.txt"
    good.write_text("# settings measured on some node\nmax_ctas = 8\nsub_max 4096   # small steps\n\nmin_steps=2\n")
    monkeypatch.setenv("HXCCL_TUNE_FILE", str(good))
    rc, (ctas, threads, steps, epochs, sub), why = plan("sliced", 64 << 20, 2, 253 << 20)
    assert rc == 0 and ctas == 8 and sub == 4096 and steps == (64 << 20) // 2 // 8 // 4096 and epochs == steps + 2
    bad = tmp_path / "bad.txt"
    bad.write_text("max_ctas 8\nno_such_knob 3\n")
    monkeypatch.setenv("HXCCL_TUNE_FILE", str(bad))
    rc, _, why = plan("sliced", 1 << 20, 2, 253 << 20)
    assert rc == L.INVALID_ARGUMENT and "no_such_knob" in why
    monkeypatch.setenv("HXCCL_TUNE_FILE", str(tmp_path / "missing.txt"))
    assert plan("sliced", 1 << 20, 2, 253 << 20)[0] == L.INVALID_ARGUMENT


def choose(nbytes, dt, n, exact=1, nvls=1):
    lib = L.lib()
    lib.hxcclTestChooseVariant.argtypes = [C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int),
                                           C.POINTER(C.c_int), C.POINTER(C.c_size_t)]
    v, tab = C.c_int(), C.c_int()
    shape = (C.c_size_t * 3)()
    rc = lib.hxcclTestChooseVariant(nbytes, dt, n, exact, nvls, C.byref(v), C.byref(tab), shape)
    return rc, v.value, bool(tab.value), list(shape)


def test_tuning_table_rows_decide_the_variant(tmp_path, monkeypatch):
    """A table row picks the AllReduce variant and its launch shape for its size range, rank
    count, element size and mode; outside the rows the fixed thresholds hold; a row that cannot
    run (multicast reduction without multicast) is skipped."""
    table = tmp_path / "table.tune"
    table.write_text(
        "# measured elsewhere\n"
        "row allreduce n=8 mode=exact from=0 variant=lines\n"
        "row allreduce n=8 mode=exact from=4096 variant=oneshot\n"
        "row allreduce n=8 mode=exact from=1048576 variant=twoshot ctas=64 sub=65536\n"
        "row allreduce n=8 es=2 mode=exact from=1048576 variant=ring ctas=200 threads=256 sub=131072\n"
        "row allreduce n=8 mode=exact from=268435456 variant=twoshot_roles\n"
        "row allreduce n=8 mode=fast from=65536 variant=nvls\n"
        "row allreduce n=4 from=0 variant=twoshot\n"
        "max_ctas 96\n")
    monkeypatch.setenv("HXCCL_TUNE_FILE", str(table))
    assert choose(8, L.FLOAT32, 8)[1:3] == (7, True)
    assert choose(8192, L.FLOAT32, 8)[1:3] == (1, True)
    rc, v, tab, shape = choose(4 << 20, L.FLOAT32, 8)
    assert (rc, v, tab, shape) == (0, 2, True, [64, 0, 65536])
    rc, v, tab, shape = choose(4 << 20, L.BFLOAT16, 8)          # the row for 2-byte elements wins
    assert (v, tab, shape) == (6, True, [200, 256, 131072])
    assert choose(1 << 30, L.FLOAT32, 8)[1:3] == (4, True)
    assert choose(1 << 20, L.FLOAT32, 8, exact=0)[1:3] == (3, True)
    assert choose(1 << 20, L.FLOAT32, 8, exact=0, nvls=0)[2] is False  # cannot run: thresholds decide
    assert choose(100, L.FLOAT32, 5)[1:3] == (2, True)           # five ranks use the rows of four
    assert choose(100, L.FLOAT32, 2)[2] is False                 # nothing tabled for two ranks
    assert choose(100, L.FLOAT32, 2)[1] == 7 and choose(1 << 20, L.FLOAT32, 2)[1] == 2
    bad = tmp_path / "bad.tune"
    bad.write_text("row allreduce n=8 from=0 variant=warp_drive\n")
    monkeypatch.setenv("HXCCL_TUNE_FILE", str(bad))
    assert choose(8, L.FLOAT32, 8)[0] == L.INVALID_ARGUMENT


def test_compiled_in_table_parses():
    """Every row of the compiled-in table is well formed: the source text and what the library
    loaded agree on the number of rows."""
    import re
    from pathlib import Path

    text = (Path(__file__).resolve().parent.parent / "src" / "device" / "tune_default.inc").read_text()
    body = text[text.index('R"TUNE(') + 7:text.index(')TUNE"')]
    rows = [ln for ln in body.splitlines() if re.match(r"\s*row\b", ln.split("#")[0])]
    lib = L.lib()
    lib.hxcclTestTableRows.restype = C.c_int
    assert lib.hxcclTestTableRows() == len(rows)


def test_explain_tool_prints_the_choice_per_size(capsys, monkeypatch):
    """python -m hxccl_b200.explain: one line per size with the variant and who decided."""
    from hxccl_b200 import explain

    monkeypatch.delenv("HXCCL_TUNE_FILE", raising=False)
    assert explain.main(["--ranks", "8", "--from", "8", "--to", "256M"]) == 0
    lines = capsys.readouterr().out.splitlines()
    assert lines[0].split()[:2] == ["bytes", "variant"] and len(lines) == 1 + 26
    first, last = lines[1].split(), lines[-1].split()
    assert first[:2] == ["8", "lines"] and last[:2] == [str(256 << 20), "ring"]
    name, tabled, shape = explain.choose(100, L.FLOAT32, 3)  # three ranks use the rows measured for two
    assert name in explain.VARIANTS.values() and len(shape) == 3
    with pytest.raises(ValueError):
        explain.choose(100, L.FLOAT32, 1)
