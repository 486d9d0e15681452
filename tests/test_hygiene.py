"""Static hygiene checks over the source tree (the reference runs similar scripts as unit tests:
scripts/check_no_default_stream_in_gpu_code.sh, scripts/check_no_direct_getenv.sh)."""
import pathlib
import re

ROOT = pathlib.Path(__file__).resolve().parents[1]
PKG = ROOT / "llaminar_b200"


def _sources(*suffixes):
    for p in list(PKG.rglob("*")) + [ROOT / "bench.py", ROOT / "__graft_entry__.py"] + list((ROOT / "tests").glob("*.py")):
        if p.is_file() and p.suffix in suffixes and "_build" not in p.parts:
            yield p


def test_no_direct_reads_of_llaminar_environment_switches():
    bad = []
    for p in _sources(".py"):
        if p.name in ("env.py", "test_hygiene.py"):
            continue
        for i, line in enumerate(p.read_text().splitlines(), 1):
            if re.search(r"environ(\.get)?[\[(]\s*[\"']LLAMINAR_", line):
                bad.append(f"{p.relative_to(ROOT)}:{i}")
    assert not bad, f"read LLAMINAR_* switches through utils.env.debug_env(): {bad}"


def test_every_kernel_launch_names_its_stream():
    bad = []
    for p in _sources(".cu", ".cuh"):
        for m in re.finditer(r"<<<(.*?)>>>", p.read_text(), flags=re.S):
            depth, args, cur = 0, [], ""
            for ch in m.group(1):
                if ch in "(<":
                    depth += 1
                elif ch in ")>":
                    depth -= 1
                if ch == "," and depth == 0:
                    args.append(cur)
                    cur = ""
                else:
                    cur += ch
            args.append(cur)
            if len(args) < 4:
                bad.append(f"{p.name}: <<<{m.group(1)[:40]}>>>")
    assert not bad, f"kernel launches without an explicit stream: {bad}"


def test_no_cuda_malloc_on_the_hot_path():
    bad = [p.name for p in _sources(".cu", ".cuh", ".cpp") if re.search(r"\bcudaMalloc\w*\s*\(", p.read_text())]
    assert not bad, f"device allocations belong to torch's allocator, found cudaMalloc in {bad}"


def test_every_registered_switch_is_documented_and_typed():
    from llaminar_b200.utils.env import REGISTRY, DebugEnv
    names = [e.name for e in REGISTRY]
    assert len(names) == len(set(names)) and all(n.startswith("LLAMINAR_") and e.help for n, e in zip(names, REGISTRY))
    env = DebugEnv({"LLAMINAR_TP_FUSED": "0", "LLAMINAR_HEARTBEAT_S": "0.5", "LLAMINAR_TYPO": "1"})
    assert env.tp_fused is False and env.heartbeat_s == 0.5 and env.unknown() == ["LLAMINAR_TYPO"]


def test_comments_stand_on_their_own():
    """Source files do not point at build notes, machine paths or tooling of the build environment."""
    banned = re.compile(r"SURVEY|VERDICT|ADVICE\.md|DESIGN\.md|BASELINE\.md|gpurun|/root/")
    bad = []
    for p in _sources(".py", ".cu", ".cuh", ".cpp", ".h"):
        if p.name == "test_hygiene.py":
            continue
        for i, line in enumerate(p.read_text().splitlines(), 1):
            if banned.search(line):
                bad.append(f"{p.relative_to(ROOT)}:{i}: {line.strip()[:80]}")
    assert not bad, bad
