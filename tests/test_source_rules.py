"""Static checks on the shipped sources: the product never touches the oracle, and every
polling site in the kernels sits next to an iteration limit."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SOURCE_EXT = (".cu", ".cuh", ".hpp", ".h", ".cpp", ".c", ".py")
SKIP_DIRS = {"__pycache__", "build"}


def test_product_never_reaches_the_oracle():
    # the oracle is test infrastructure: the package must not import, load or link it
    pkg = os.path.join(ROOT, "cortexsdr_b200")
    rx = re.compile(r"\boracle\b|hsdr_oracle|libcortexsdr_ref")
    hits = []
    for base, dirs, files in os.walk(pkg):
        dirs[:] = [d for d in dirs if d not in SKIP_DIRS]
        for f in files:
            if not f.endswith(SOURCE_EXT + ("Makefile",)):
                continue
            path = os.path.join(base, f)
            with open(path, errors="replace") as fh:
                for n, line in enumerate(fh, 1):
                    code = line.split("//")[0].split("#")[0]
                    if rx.search(code):
                        hits.append(f"{os.path.relpath(path, ROOT)}:{n}: {line.strip()}")
    assert hits == []


def test_device_waits_are_bounded():
    # every polling site in the kernels (an mbarrier try_wait, a system-scope acquire load of a
    # flag, a loop without an exit condition) sits next to an iteration limit
    kdir = os.path.join(ROOT, "cortexsdr_b200", "csrc", "kernels")
    poll = re.compile(r"mbarrier\.try_wait|while\s*\(\s*ld_acquire|while\s*\(\s*(true|1)\s*\)|for\s*\([^;]*;\s*;")
    bound = re.compile(r"[sS]pin|limit|Limit")
    sites, unbounded = 0, []
    for f in sorted(os.listdir(kdir)):
        if not f.endswith((".cu", ".cuh")):
            continue
        lines = open(os.path.join(kdir, f), errors="replace").read().splitlines()
        for n, line in enumerate(lines):
            if line.lstrip().startswith("//") or not poll.search(line):
                continue
            sites += 1
            window = "\n".join(lines[max(0, n - 8):n + 24])
            if not bound.search(window):
                unbounded.append(f"{f}:{n + 1}")
    assert sites >= 4          # the check sees the waits it is meant to see
    assert unbounded == []
