"""Static audits of the CUDA sources (no GPU): every kernel orders itself after its predecessor before it touches
memory (programmatic dependent launch turns stream order into an explicit wait), no kernel traps or asserts, every
spin loop on a flag / barrier is bounded, and nothing names the closed batched-copy runtime calls.
(Model of the reference's tests/python/pdl_wait_audit.py.)"""
import glob
import os
import re

ROOT = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "dgpp_b200", "csrc")


def _sources():
    out = []
    for pat in ("**/*.cu", "**/*.cuh"):
        out += glob.glob(os.path.join(ROOT, pat), recursive=True)
    return sorted(out)


def _kernels(text):
    for m in re.finditer(r"__global__\s+void\s+(?:__launch_bounds__\([^)]*(?:\([^)]*\)[^)]*)*\)\s*)?(\w+)\s*\(", text):
        i = text.find("{", m.end())
        depth, j = 0, i
        while True:
            if text[j] == "{":
                depth += 1
            elif text[j] == "}":
                depth -= 1
                if depth == 0:
                    break
            j += 1
        yield m.group(1), text[i:j]


def test_every_kernel_waits_for_its_predecessor():
    missing, seen = [], 0
    for path in _sources():
        for name, body in _kernels(open(path).read()):
            seen += 1
            if "pdl_wait()" not in body and "griddepcontrol.wait" not in body:
                missing.append(f"{os.path.basename(path)}:{name}")
    assert seen >= 30 and not missing, missing


def test_no_traps_asserts_or_unbounded_spins():
    bad = []
    for path in _sources():
        text = open(path).read()
        code = re.sub(r"//[^\n]*", "", text)
        if re.search(r"__trap\s*\(|\bassert\s*\(|asm[^;]*\btrap;", code):
            bad.append(os.path.basename(path) + ": trap/assert")
        # a `for (;;)` or `while (true)` in device code must contain a way out that does not depend on the waited value
        for m in re.finditer(r"(for\s*\(\s*;\s*;\s*\)|while\s*\(\s*(true|1)\s*\))\s*\{", code):
            depth, j = 0, code.find("{", m.start())
            start = j
            while True:
                if code[j] == "{":
                    depth += 1
                elif code[j] == "}":
                    depth -= 1
                    if depth == 0:
                        break
                j += 1
            body = code[start:j]
            if not re.search(r"clock64|globaltimer|spins|tries|iters|budget|return|break", body):
                bad.append(f"{os.path.basename(path)}: unbounded loop near byte {m.start()}")
    assert not bad, bad


def test_closed_runtime_calls_are_not_named():
    names = ["cudaMemcpy" + "BatchAsync", "cudaMemcpy3D" + "BatchAsync", "cuMemcpy" + "BatchAsync", "cuMemcpy3D" + "BatchAsync"]
    repo = os.path.dirname(os.path.dirname(ROOT))
    hits = []
    roots = [os.path.join(repo, d) for d in ("dgpp_b200", "tests", "deploy")]
    walk = [(repo, [], [f for f in os.listdir(repo) if os.path.isfile(os.path.join(repo, f))])]
    for r in roots:
        walk += [(dp, dn, fs) for dp, dn, fs in os.walk(r) if "__pycache__" not in dp and os.sep + "build" not in dp]
    for dirpath, dirnames, files in walk:
        for f in files:
            if f.endswith((".cu", ".cuh", ".h", ".cpp", ".py", ".sh")):
                text = open(os.path.join(dirpath, f), errors="ignore").read()
                hits += [f"{f}: {n}" for n in names if n in text]
    assert not hits, hits


def test_no_cluster_multicast_loads():
    """No TMA / bulk LOAD carries the cluster-multicast qualifier (a commit that arrives on the barriers of a CTA pair
    may: it moves no data)."""
    hits = []
    pat = re.compile(r"cp\.async\.bulk[^;\n]*" + re.escape(".multi" + "cast::" + "cluster"))
    for path in _sources():
        if pat.search(open(path).read()):
            hits.append(os.path.basename(path))
    assert not hits, hits
