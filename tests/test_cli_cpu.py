"""Launcher: resolve (strict keys, site defaults, overrides, digest), doctor on a box without GPUs, and a full
up / status / down cycle of the fake-engine deployment.  (Model of the reference's tests/python/test_cluster_cli.py
with its fake SSH; here everything is local.)"""
import json
import os
import socket

import pytest

from dgpp_b200 import cli

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_resolve_defaults_overrides_and_unknown_keys(tmp_path):
    dep = tmp_path / "d.json"
    dep.write_text(json.dumps({"model": "fake", "max_concurrency": 2}))
    env = tmp_path / "site.env"
    env.write_text("# comment\nHOST=10.0.0.5\nPORT=9001\nLOG_LEVEL=debug\n")
    cfg, d1 = cli.resolve(str(dep), str(env))
    assert (cfg["host"], cfg["port"], cfg["log_level"], cfg["max_concurrency"]) == ("10.0.0.5", 9001, "debug", 2)
    cfg2, d2 = cli.resolve(str(dep), str(env), ["port=9100", "prefix_cache=false"])
    assert cfg2["port"] == 9100 and cfg2["prefix_cache"] is False and d1 != d2
    assert cli.resolve(str(dep), str(env))[1] == d1                      # the digest is a function of the config
    dep.write_text(json.dumps({"model": "fake", "max_concurency": 2}))
    with pytest.raises(RuntimeError, match="unknown key"):
        cli.resolve(str(dep))
    # the shipped templates resolve
    for name in os.listdir(os.path.join(ROOT, "deploy")):
        if name.endswith(".json"):
            cli.resolve(os.path.join(ROOT, "deploy", name))


def test_model_root_lookup(tmp_path):
    (tmp_path / "models" / "org" / "m").mkdir(parents=True)
    dep = tmp_path / "d.json"
    dep.write_text(json.dumps({"model": "org/m"}))
    env = tmp_path / "site.env"
    env.write_text(f"MODEL_ROOT={tmp_path / 'models'}\n")
    assert cli.resolve(str(dep), str(env))[0]["model"] == str(tmp_path / "models" / "org" / "m")
    assert cli.resolve(str(dep))[0]["model"] == "org/m"


def test_doctor_reports_without_gpus(tmp_path):
    rows, ok = cli.doctor(str(tmp_path))
    names = {r[0]: r for r in rows}
    assert names["kernel library"][1] and names["runtime module"][1] and names["runtime import"][1]
    assert "ok" in names["runtime import"][2] and names["cache dir"][1]
    assert ok                                                            # missing GPUs are reported, not fatal


def test_up_status_down_cycle(tmp_path):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    dep = tmp_path / "d.json"
    dep.write_text(json.dumps({"model": "fake", "port": port, "max_concurrency": 2, "log_level": "warn"}))
    run = str(tmp_path / "run")
    r = cli.up(str(dep), run, wait_s=90)
    try:
        assert r["healthy"], open(r["log"]).read()[-2000:]
        with pytest.raises(RuntimeError, match="still running"):
            cli.up(str(dep), run)
        st = cli.status(run)
        assert st["running"] and st["health"] == {"status": "ok"} and "requests_total" in st["counters"]
    finally:
        d = cli.down(run)
    assert d["stopped"] and not cli._pid_alive(d["pid"])
    assert cli.status(run) == {"running": False, "reason": "no pid file"}
