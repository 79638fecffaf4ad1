"""``areno env`` / ``areno check``: the report's shape, every PASS / WARN / FAIL rule on synthetic reports, and the CLI."""

from __future__ import annotations

import copy
import json

from click.testing import CliRunner

from areno_b200.cli import diagnostics as dg


def _report(**over):
    base = {
        "areno_b200": {"version": "0.1"}, "python": {"version": "3.12.3", "executable": "/usr/bin/python"},
        "platform": {"system": "Linux", "release": "6", "machine": "x86_64"},
        "torch": {"imported": True, "version": "2.11", "cuda_build": "12.8", "cuda_available": True, "nccl": "2.28"},
        "cuda": {"cuda_home": None, "nvcc": {"path": "/usr/local/cuda/bin/nvcc", "version": "12.9.86"},
                 "driver": {"driver_version": "580.1"}},
        "gpus": [{"index": 0, "name": "NVIDIA B200", "capability": "10.0", "memory_gb": 179.1, "sm_count": 148}],
        "native": {"kernels": {"path": "/x/libareno_kernels.so", "built": True, "size_bytes": 1},
                   "runtime": {"path": "/x/libareno_runtime.so", "built": True, "size_bytes": 1}},
        "dependencies": {"transformers": "5", "safetensors": "0.5", "datasets": None, "fastapi": "1", "uvicorn": "1",
                         "tensorboard": None, "click": "8"},
        "env": {"ARENO_LOG_LEVEL": None}, "paths": {"metrics_log_dir": "/tmp/areno/tfevent", "hf_cache": "/tmp/hf"},
    }
    rep = copy.deepcopy(base)
    for key, val in over.items():
        node = rep
        *parents, leaf = key.split(".")
        for p in parents:
            node = node[p]
        node[leaf] = val
    return rep


def _status(rows, name):
    return next(r for r in rows if r.name.startswith(name)).status


def test_version_tuple_parses_dotted_versions_with_suffixes():
    assert dg._version_tuple("12.9.86") == (12, 9, 86) and dg._version_tuple("12.8rc1") == (12, 8)
    assert dg._version_tuple(None) == () and dg._version_tuple("abc") == ()


def test_a_ready_machine_passes_with_warnings_only_for_optional_packages():
    rows = dg.run_checks(_report())
    assert not [r for r in rows if r.status == "FAIL"]
    assert _status(rows, "datasets installed") == "WARN" and _status(rows, "GPUs are sm_100") == "PASS"
    assert all(r.next_step for r in rows if r.status != "PASS")


def test_hard_requirements_fail_and_soft_ones_warn():
    rows = dg.run_checks(_report(**{"torch.cuda_available": False, "gpus": [], "torch.nccl": None,
                                    "dependencies.transformers": None, "cuda.driver.driver_version": None}))
    assert _status(rows, "CUDA device visible") == "FAIL" and _status(rows, "transformers installed") == "FAIL"
    assert _status(rows, "NCCL available") == "WARN" and _status(rows, "NVIDIA driver reported") == "WARN"
    assert not [r for r in rows if r.name.startswith("GPUs are sm_100")]          # no GPU row without GPUs


def test_other_gpu_generations_are_rejected():
    h100 = [{"index": 0, "name": "NVIDIA H100", "capability": "9.0", "memory_gb": 80.0, "sm_count": 132}]
    assert _status(dg.run_checks(_report(gpus=h100)), "GPUs are sm_100") == "FAIL"


def test_old_or_missing_nvcc_only_warns_while_prebuilt_libraries_exist():
    old = {"path": "/usr/bin/nvcc", "version": "12.4"}
    assert _status(dg.run_checks(_report(**{"cuda.nvcc": old})), "nvcc >= 12.8") == "WARN"
    rep = _report(**{"cuda.nvcc": {"path": None, "version": None}})
    rep["native"]["kernels"]["built"] = False
    rows = dg.run_checks(rep)
    assert _status(rows, "nvcc >= 12.8") == "FAIL" and _status(rows, "native kernels library built") == "FAIL"


def test_unwritable_directories_warn(tmp_path):
    locked = tmp_path / "ro"
    locked.mkdir()
    locked.chmod(0o500)
    try:
        row = dg._writable("metrics_log_dir", str(locked / "a" / "b"))
        import os
        if os.geteuid() != 0:            # root can write anywhere: the rule cannot trigger
            assert row.status == "WARN" and str(locked) in row.detail
        assert dg._writable("metrics_log_dir", str(tmp_path / "new" / "dir")).status == "PASS"
    finally:
        locked.chmod(0o700)


def test_text_report_lists_gpus_libraries_and_environment():
    text = dg.format_env_report(_report())
    assert "NVIDIA B200  sm_10.0  179.1 GiB  148 SMs" in text and "kernels  built" in text
    assert "datasets      not installed" in text and "ARENO_LOG_LEVEL=" in text
    assert "none visible" in dg.format_env_report(_report(gpus=[]))


def test_collect_env_has_every_section_on_this_machine():
    rep = dg.collect_env()
    assert {"areno_b200", "python", "platform", "torch", "cuda", "gpus", "native", "dependencies", "env", "paths"} <= set(rep)
    assert set(rep["native"]) == {"kernels", "runtime"} and rep["torch"]["imported"] is True


def test_env_command_emits_json_and_text():
    out = CliRunner().invoke(dg.env_command, ["--json"])
    assert out.exit_code == 0 and "torch" in json.loads(out.output)
    assert "AReno-B200 environment" in CliRunner().invoke(dg.env_command, []).output
