"""Launcher for one 8 x B200 box: ``python -m dgpp_b200.cli <command>``.

    resolve  <deployment.json> [--env FILE] [--set key=value ...]   effective config (strict keys) + digest
    doctor   [--cache-dir DIR]                                       environment report; exit 1 when a check fails
    up       <deployment.json> [--run-dir DIR]                       start the server in the background
    status   [--run-dir DIR]                                         process + /health + /metrics summary
    down     [--run-dir DIR]                                         stop the server this launcher started

Deployment JSON keys are the server's own (unknown keys are errors, see ``rt.parse_cluster_config``); a site ``.env``
file supplies defaults for HOST / PORT / LOG_LEVEL / MODEL_ROOT (a relative ``model`` is resolved under MODEL_ROOT).
`up` writes ``server.pid``, ``server.log`` and ``resolved.json`` into the run directory; `down` signals exactly the
recorded process id, never a name pattern.
(reference counterparts: scripts/dgpp-cluster up / down / status / resolve / doctor, scripts/cluster_doctor.py,
 scripts/site_env.py -- there over SSH to several nodes, here one box.)
"""
from __future__ import annotations

import argparse
import json
import os
import resource
import signal
import subprocess
import sys
import time
import urllib.request
from typing import Dict, List, Tuple

DEFAULT_RUN_DIR = os.path.join(os.path.expanduser("~"), ".dgpp_b200", "run")


def read_env_file(path: str) -> Dict[str, str]:
    out: Dict[str, str] = {}
    if not path or not os.path.exists(path):
        return out
    for line in open(path):
        line = line.strip()
        if not line or line.startswith("#") or "=" not in line:
            continue
        k, v = line.split("=", 1)
        out[k.strip()] = v.strip().strip('"').strip("'")
    return out


def resolve(deployment_path: str, env_path: str = "", overrides: List[str] = ()) -> Tuple[dict, int]:
    """Deployment JSON + site defaults + command-line overrides -> (effective config, digest)."""
    from .runtime import rt

    dep = json.load(open(deployment_path))
    if not isinstance(dep, dict):
        raise ValueError("deployment: the top level must be an object")
    env = read_env_file(env_path)
    for key, env_key, cast in (("host", "HOST", str), ("port", "PORT", int), ("log_level", "LOG_LEVEL", str)):
        if key not in dep and env_key in env:
            dep[key] = cast(env[env_key])
    for item in overrides:
        if "=" not in item:
            raise ValueError(f"--set wants key=value, got {item!r}")
        k, v = item.split("=", 1)
        try:
            dep[k] = json.loads(v)
        except ValueError:
            dep[k] = v
    model = dep.get("model", "")
    root = env.get("MODEL_ROOT", "")
    if root and model and model not in ("fake", "tiny") and not os.path.isabs(model) and os.path.isdir(os.path.join(root, model)):
        dep["model"] = os.path.join(root, model)
    text, digest = rt.parse_cluster_config(json.dumps(dep))
    return json.loads(text), digest


def doctor(cache_dir: str = "") -> Tuple[List[Tuple[str, bool, str]], bool]:
    """Checks a deployment depends on.  Each row: (check, ok, detail).  Rows marked optional do not fail the run."""
    rows: List[Tuple[str, bool, str]] = []
    ok_all = True

    def add(name, ok, detail, required=True):
        nonlocal ok_all
        rows.append((name, bool(ok), detail))
        if required and not ok:
            ok_all = False

    add("python", sys.version_info >= (3, 10), sys.version.split()[0])
    try:
        import torch
        add("torch", True, torch.__version__)
    except Exception as e:  # pragma: no cover
        add("torch", False, str(e))
        return rows, False
    from . import build
    kern = build.LIB / "libdgpp_kernels.so"
    add("kernel library", kern.exists(), str(kern))
    add("runtime module", build.rt_module_path().exists(), str(build.rt_module_path()))
    try:
        from .runtime import rt
        add("runtime import", True, "crc32c self-test " + ("ok" if rt.crc32c(b"123456789") == 0xE3069283 else "FAILED"))
    except Exception as e:
        add("runtime import", False, str(e))
        rt = None
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    add("cuda devices", n > 0, f"{n} visible", required=False)
    for i in range(n):
        p = torch.cuda.get_device_properties(i)
        add(f"gpu{i}", p.major == 10, f"{p.name} sm_{p.major}{p.minor} {p.total_memory >> 30} GiB {p.multi_processor_count} SMs")
    if n > 1:
        bad = [(a, b) for a in range(n) for b in range(n) if a != b and not torch.cuda.can_device_access_peer(a, b)]
        add("peer access", not bad, "all pairs" if not bad else f"no peer access between {bad[:4]}")
    import torch.distributed as dist
    add("nccl backend", dist.is_nccl_available(), "torch.distributed", required=False)
    soft, _ = resource.getrlimit(resource.RLIMIT_MEMLOCK)
    add("memlock limit", soft == resource.RLIM_INFINITY or soft >= (1 << 30),
        "unlimited" if soft == resource.RLIM_INFINITY else f"{soft >> 20} MiB (pinned staging wants >= 1 GiB)", required=False)
    if cache_dir and rt is not None:
        info = rt.probe_cache_storage(cache_dir)
        add("cache dir", info["exists"] and info["writable"],
            f"{cache_dir}: free {info['free_bytes'] >> 30} GiB, O_DIRECT {'yes' if info['direct_io'] else 'no'}")
    return rows, ok_all


def _pid_alive(pid: int) -> bool:
    try:
        os.kill(pid, 0)
        return True
    except OSError:
        return False


def up(deployment_path: str, run_dir: str, env_path: str = "", overrides: List[str] = (), wait_s: float = 60.0) -> dict:
    cfg, digest = resolve(deployment_path, env_path, overrides)
    os.makedirs(run_dir, exist_ok=True)
    pid_path = os.path.join(run_dir, "server.pid")
    if os.path.exists(pid_path):
        old = int(open(pid_path).read().strip() or 0)
        if old and _pid_alive(old):
            raise RuntimeError(f"a server started from {run_dir} is still running (pid {old}); run `down` first")
    resolved = os.path.join(run_dir, "resolved.json")
    json.dump(cfg, open(resolved, "w"), indent=1)
    log = open(os.path.join(run_dir, "server.log"), "ab")
    env = dict(os.environ)
    env.update({k: v for k, v in read_env_file(env_path).items() if k.startswith("DGPP_")})
    proc = subprocess.Popen([sys.executable, "-m", "dgpp_b200.serve.app", "--config", resolved], stdout=log,
                            stderr=subprocess.STDOUT, env=env, start_new_session=True,
                            cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    open(pid_path, "w").write(str(proc.pid))
    url = f"http://{cfg['host']}:{cfg['port']}/health"
    deadline = time.time() + wait_s
    healthy = False
    while time.time() < deadline and proc.poll() is None:
        try:
            with urllib.request.urlopen(url, timeout=1) as r:
                healthy = r.status == 200
                break
        except OSError:
            time.sleep(0.2)
    return {"pid": proc.pid, "healthy": healthy, "exited": proc.poll(), "url": url, "digest": f"{digest:016x}",
            "log": log.name}


def status(run_dir: str) -> dict:
    pid_path = os.path.join(run_dir, "server.pid")
    if not os.path.exists(pid_path):
        return {"running": False, "reason": "no pid file"}
    pid = int(open(pid_path).read().strip() or 0)
    out = {"pid": pid, "running": bool(pid) and _pid_alive(pid)}
    try:
        cfg = json.load(open(os.path.join(run_dir, "resolved.json")))
        base = f"http://{cfg['host']}:{cfg['port']}"
        with urllib.request.urlopen(base + "/health", timeout=2) as r:
            out["health"] = json.loads(r.read())
        with urllib.request.urlopen(base + "/metrics", timeout=2) as r:
            out["counters"] = json.loads(r.read()).get("counters", {})
    except (OSError, ValueError) as e:
        out["health"] = f"unreachable: {e}"
    return out


def down(run_dir: str, grace_s: float = 30.0) -> dict:
    pid_path = os.path.join(run_dir, "server.pid")
    if not os.path.exists(pid_path):
        return {"stopped": False, "reason": "no pid file"}
    pid = int(open(pid_path).read().strip() or 0)
    if pid and _pid_alive(pid):
        os.kill(pid, signal.SIGINT)                      # the server's own orderly shutdown path
        deadline = time.time() + grace_s
        while time.time() < deadline and _pid_alive(pid):
            try:
                os.waitpid(pid, os.WNOHANG)              # reap it when it is our child
            except ChildProcessError:
                pass
            time.sleep(0.1)
        if _pid_alive(pid):
            os.kill(pid, signal.SIGKILL)
    os.remove(pid_path)
    return {"stopped": True, "pid": pid}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="dgpp_b200.cli", description=__doc__.split("\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name in ("resolve", "up"):
        p = sub.add_parser(name)
        p.add_argument("deployment")
        p.add_argument("--env", default="")
        p.add_argument("--set", action="append", default=[], dest="overrides")
        if name == "up":
            p.add_argument("--run-dir", default=DEFAULT_RUN_DIR)
    p = sub.add_parser("doctor")
    p.add_argument("--cache-dir", default="")
    for name in ("status", "down", "metrics", "api-check"):
        p = sub.add_parser(name)
        p.add_argument("--run-dir", default=DEFAULT_RUN_DIR)
        if name == "metrics":
            p.add_argument("--prometheus", action="store_true")
    a = ap.parse_args(argv)
    if a.cmd in ("metrics", "api-check"):
        # the running deployment's own endpoints (its address comes from the run directory's resolved config)
        cfg = json.load(open(os.path.join(a.run_dir, "resolved.json")))
        base = f"http://{cfg['host']}:{cfg['port']}"
        if a.cmd == "api-check":
            from .tools import api_check
            return api_check.main(["--url", base])
        with urllib.request.urlopen(base + ("/metrics/prometheus" if a.prometheus else "/metrics"), timeout=5) as r:
            body = r.read().decode()
        print(body if a.prometheus else json.dumps(json.loads(body), indent=1))
        return 0
    if a.cmd == "resolve":
        cfg, digest = resolve(a.deployment, a.env, a.overrides)
        print(json.dumps({"config": cfg, "digest": f"{digest:016x}"}, indent=1))
        return 0
    if a.cmd == "doctor":
        rows, ok = doctor(a.cache_dir)
        for name, good, detail in rows:
            print(f"{'ok  ' if good else 'FAIL'} {name:16s} {detail}")
        return 0 if ok else 1
    if a.cmd == "up":
        r = up(a.deployment, a.run_dir, a.env, a.overrides)
        print(json.dumps(r, indent=1))
        return 0 if r["healthy"] else 1
    if a.cmd == "status":
        print(json.dumps(status(a.run_dir), indent=1))
        return 0
    print(json.dumps(down(a.run_dir), indent=1))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
