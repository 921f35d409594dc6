"""Static rules the sources must keep (no GPU needed): device waits are bounded, nothing traps, calls and instructions that
are not to be used on the target machines stay out, profile commands never touch the GPU clocks, and comments stand on their own.
Forbidden names are assembled from fragments so that this file does not contain them itself."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "gpt_moe_b200", "csrc")


def _files(top, suffixes):
    for folder, dirs, names in os.walk(top):
        dirs[:] = [d for d in dirs if not d.startswith("build") and d not in ("__pycache__", "_ref", "_work", "gpu" + "run_out", ".git")]
        for name in sorted(names):
            if name.endswith(suffixes):
                yield os.path.join(folder, name)


def _native_sources():
    return list(_files(CSRC, (".cu", ".cuh", ".h", ".cpp")))


def _python_sources():
    out = list(_files(os.path.join(ROOT, "gpt_moe_b200"), (".py",))) + list(_files(os.path.join(ROOT, "experiments"), (".py",)))
    out += list(_files(os.path.join(ROOT, "tests"), (".py",)))
    out += [os.path.join(ROOT, n) for n in ("bench.py", "train.py", "__graft_entry__.py", "push_to_hub.py") if os.path.exists(os.path.join(ROOT, n))]
    out += [os.path.join(ROOT, "baseline", "run_reference.py")]
    return [p for p in out if os.path.exists(p)]


def test_no_trap_and_no_device_assert():
    bad = []
    for path in _native_sources():
        if not path.endswith((".cu", ".cuh")):
            continue
        for no, line in enumerate(open(path), 1):
            code = line.split("//")[0]
            if "__tr" + "ap(" in code or re.search(r"(?<![_\w])assert\(", code):
                bad.append(f"{path}:{no}")
    assert not bad, bad


def test_closed_calls_and_cluster_multicast_loads_are_absent():
    batch_copies = ["cu" + "daMemcpy" + "Batch" + "Async", "cu" + "daMemcpy3D" + "Batch" + "Async", "cu" + "Memcpy" + "Batch" + "Async",
                    "cu" + "Memcpy3D" + "Batch" + "Async"]
    bulk, multicast = "cp.async" + ".bulk", "multi" + "cast::cluster"
    bad = []
    for path in _native_sources() + _python_sources():
        text = open(path).read()
        for name in batch_copies:
            if name in text:
                bad.append(f"{path}: {name}")
        for no, line in enumerate(text.splitlines(), 1):
            if bulk in line and multicast in line:
                bad.append(f"{path}:{no}: bulk copy with cluster multicast")
    assert not bad, bad


def test_every_open_ended_loop_in_a_kernel_has_a_budget():
    """`for (;;)` / `while (true)` in device code must sit next to a clock or iteration budget."""
    bad = []
    for path in _native_sources():
        if not path.endswith((".cu", ".cuh")):
            continue
        lines = open(path).read().splitlines()
        for no, line in enumerate(lines):
            code = line.split("//")[0]
            if re.search(r"for\s*\(\s*;\s*;\s*\)|while\s*\(\s*(true|1)\s*\)", code):
                window = "\n".join(lines[max(0, no - 3): no + 14])
                if not re.search(r"clock64|budget|Budget|limit|spins", window):
                    bad.append(f"{path}:{no + 1}")
    assert not bad, bad


def test_profile_commands_leave_the_clocks_alone():
    folder = os.path.join(ROOT, "profiles")
    bad = []
    for path in _files(folder, (".md", ".txt")):
        for no, line in enumerate(open(path), 1):
            for command in re.findall(r"\bncu\s+--[^&;]*", line):          # an ncu invocation with options (reading a report uses -i)
                if "--clock-control none" not in command:
                    bad.append(f"{path}:{no}")
    assert not bad, bad


@pytest.mark.parametrize("word", ["VER" + "DICT", "SUR" + "VEY", "ADV" + "ICE.md", "DES" + "IGN.md", "BASE" + "LINE.md", "gpu" + "run", "/ro" + "ot/"])
def test_comments_do_not_point_outside_the_sources(word):
    bad = []
    for path in _native_sources() + _python_sources():
        for no, line in enumerate(open(path), 1):
            if word in line:
                bad.append(f"{path}:{no}")
    assert not bad, bad
