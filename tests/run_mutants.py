#!/usr/bin/env python3
"""Applies every mutant of tests/mutants.txt to a scratch copy of the repository, one at a time,
and runs the test named beside it there: the test must fail.  First the same tests run on the
unchanged copy and must pass.  Prints one line per mutant; exits 1 if a mutant survives or the
baseline is red.  (The reference's counterpart: tests/lfm25_negative_controls.sh over
tests/lfm25_negctl.txt.)

    python tests/run_mutants.py [--only NAME ...] [--keep]

Mutated kernels are compiled into the scratch copy (TUFF_BUILD_DIR points there), never into the
tree.  GPU tests need a GPU; mutants whose test is a CPU test run anywhere (--cpu runs only those).
"""
import argparse
import os
import shutil
import subprocess
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CPU_TESTS = ("tests/test_scheduler.py", "tests/test_cache_manager.py", "tests/test_config_weights.py", "tests/test_plain.py", "tests/test_index_helpers.py")


def untracked_patterns():
    """What .gitignore lists (built files, caches, scratch folders): none of it belongs in the scratch copy."""
    out = []
    with open(os.path.join(ROOT, ".gitignore")) as f:
        for line in f:
            line = line.strip()
            if line and not line.startswith("#"):
                out.append(line.strip("/").split("/")[0])
    return out


def read_mutants(path):
    out, cur = [], None
    with open(path) as f:
        for raw in f:
            line = raw.rstrip("\n")
            if line.startswith("@"):
                parts = [p.strip() for p in line[1:].split("|")]
                cur = dict(name=parts[0], file=parts[1], test=parts[2], select=parts[3] if len(parts) > 3 else "",
                           old=None, new=None)
                out.append(cur)
            elif line.startswith("- ") and cur is not None and cur["old"] is None:
                cur["old"] = line[2:]
            elif line.startswith("+ ") and cur is not None and cur["new"] is None:
                cur["new"] = line[2:]
    for m in out:
        if m["old"] is None or m["new"] is None or m["old"] == m["new"]:
            raise SystemExit(f"mutant {m['name']}: needs a '- old' and a different '+ new' line")
    return out


def run_test(copy, m, timeout=1200):
    env = dict(os.environ, PYTHONPATH=copy, TUFF_BUILD_DIR=os.path.join(copy, "_mutant_build"))
    cmd = [sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider", m["test"]]
    if m["select"]:
        cmd += ["-k", m["select"]]
    proc = subprocess.run(cmd, cwd=copy, env=env, capture_output=True, text=True, timeout=timeout)
    tail = (proc.stdout + proc.stderr).strip().splitlines()[-1:] or [""]
    return proc.returncode, tail[0]


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--only", nargs="*", default=None, help="names of the mutants to run (default: all)")
    ap.add_argument("--cpu", action="store_true", help="only the mutants whose test needs no GPU")
    ap.add_argument("--keep", action="store_true", help="keep the scratch copy")
    a = ap.parse_args()
    mutants = read_mutants(os.path.join(ROOT, "tests", "mutants.txt"))
    if a.only is not None:
        mutants = [m for m in mutants if m["name"] in a.only]
    if a.cpu:
        mutants = [m for m in mutants if m["test"].split("::")[0] in CPU_TESTS]
    scratch = tempfile.mkdtemp(prefix="tuff_mutants_")
    copy = os.path.join(scratch, "repo")
    shutil.copytree(ROOT, copy, ignore=shutil.ignore_patterns(".git", *untracked_patterns()))
    bad = 0
    try:
        # the baseline: every named test passes on the unchanged copy
        seen = set()
        for m in mutants:
            key = (m["test"], m["select"])
            if key in seen:
                continue
            seen.add(key)
            rc, tail = run_test(copy, m)
            print(f"baseline  {m['test']} {('-k ' + repr(m['select'])) if m['select'] else ''}: {'passes' if rc == 0 else 'FAILS'}  [{tail}]", flush=True)
            bad += rc != 0
        if bad:
            print("the baseline is red: no mutant was run")
            return 1
        for m in mutants:
            path = os.path.join(copy, m["file"])
            with open(path) as f:
                text = f.read()
            n = text.count(m["old"])
            if n == 0:
                print(f"mutant    {m['name']}: its old text is not in {m['file']} (the table is stale)", flush=True)
                bad += 1
                continue
            with open(path, "w") as f:
                f.write(text.replace(m["old"], m["new"]))
            try:
                rc, tail = run_test(copy, m)
            finally:
                with open(path, "w") as f:
                    f.write(text)
            caught = rc != 0
            print(f"mutant    {m['name']} ({m['file']}, {n} place{'s' if n > 1 else ''}): "
                  f"{'caught by' if caught else 'SURVIVES'} {m['test']}  [{tail}]", flush=True)
            bad += not caught
    finally:
        if a.keep:
            print("scratch copy kept at", copy)
        else:
            shutil.rmtree(scratch, ignore_errors=True)
    print(f"{len(mutants)} mutants, {bad} problem(s)")
    return 1 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
