"""Static checks on the sources and the command-line contracts that need no GPU."""
import json
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC_DIRS = ("csrc", "fast_b200", "tests", "baseline")
SRC_EXT = (".cu", ".cuh", ".cc", ".cpp", ".h", ".py", ".sh")


def _ignored_dirs():
    """Directory names that version control ignores (built trees, caches, scratch), plus the history itself."""
    names = {".git", "__pycache__"}
    for line in open(os.path.join(ROOT, ".gitignore"), errors="ignore"):
        line = line.strip()
        if line.endswith("/") and "*" not in line:
            names.add(line.strip("/").split("/")[-1])
    return names


def _sources():
    for d in SRC_DIRS + ("",):
        base = os.path.join(ROOT, d)
        for dirpath, dirs, files in os.walk(base):
            dirs[:] = [x for x in dirs if x not in _ignored_dirs()]
            if d == "" and dirpath != ROOT:
                continue
            for f in files:
                if f.endswith(SRC_EXT):
                    yield os.path.join(dirpath, f)


def test_tensor_copies_stay_plain():
    """The only instruction that may carry the cluster-wide qualifier is the tensor-core commit."""
    needle = "multi" + "cast" + "::" + "cluster"
    bad = []
    for path in _sources():
        for n, line in enumerate(open(path, errors="ignore"), 1):
            if needle in line and "tcgen05.commit" not in line:
                bad.append(f"{path}:{n}")
    assert not bad, bad


def test_no_batched_memcpy_calls_are_named():
    names = [re.compile(p) for p in (r"cudaMemcpy" + r"BatchAsync", r"cudaMemcpy3D" + r"BatchAsync", r"cuMemcpy" + r"BatchAsync", r"cuMemcpy3D" + r"BatchAsync")]
    for path in _sources():
        text = open(path, errors="ignore").read()
        assert not any(r.search(text) for r in names), path


def test_every_device_wait_is_bounded():
    """Spin loops in kernels go through the bounded helpers; no bare `while (true)` / `for (;;)` polls."""
    for path in _sources():
        if not path.endswith((".cu", ".cuh")) or path.endswith("device_sync.cuh"):
            continue
        text = open(path, errors="ignore").read()
        assert "while (true)" not in text and "for (;;)" not in text and "__trap" not in text, path


def test_reference_arm_prints_unavailable_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-1000:]
    j = json.loads(r.stdout.strip().splitlines()[-1])
    assert j["impl"] == "reference" and isinstance(j["unavailable"], str) and "\n" not in j["unavailable"]


def test_graft_entry_has_build_and_smoke():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as g

    assert callable(g.build) and callable(g.smoke)
    g.build()  # up-to-date build is a no-op; a stale one recompiles for sm_100a
    import fast_b200

    assert os.path.exists(os.path.join(ROOT, "build", "fastb-sim"))
    assert any(f.startswith("_C.") and f.endswith(".so") for f in os.listdir(os.path.dirname(fast_b200.__file__)))


def test_bench_clock_sampler_parses_samples_inside_the_window():
    import importlib.util
    import time

    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)

    class _Proc:
        def terminate(self):
            pass

        def wait(self, timeout=None):
            return 0

    s = bench.ClockSampler(0)
    s.proc = _Proc()
    t0 = time.monotonic()
    s.t_begin, s.t_end = t0 + 1.0, t0 + 2.0
    row = lambda mhz, cap: [str(mhz), "1965", "640.5", "Not Active", "Not Active", "Not Active", cap]
    s.rows = [(t0 + 0.5, row(1900, "Not Active")),           # before the window: ignored
              (t0 + 1.2, row(1200, "Active")), (t0 + 1.5, row(1300, "Active")), (t0 + 1.9, row(1250, "Not Active")),
              (t0 + 1.6, ["garbage"]), (t0 + 3.0, row(1950, "Not Active"))]
    out = s.stop()
    assert out["sm_mhz"] == 1250 and out["sm_max_mhz"] == 1965 and out["samples"] == 3 and out["reasons"] == ["sw_power_cap"]
    assert out["power_w_max"] == 640.5
    s2 = bench.ClockSampler(0)                                # nvidia-smi missing: says so instead of failing
    assert s2.stop()["reasons"] == ["nvidia-smi unavailable"]
