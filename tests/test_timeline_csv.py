"""The tracing CSV is the reference's (host/net.h:539-611): its own timeline tool must read what this
runtime writes.  The writer is host code, so the file format is checked here without a GPU; the tool is
copied out of the reference tree at test time (skipped when that tree is absent)."""
import json
import os
import shutil
import subprocess
import sys

import pytest

from onenew_b200 import net as onet

TOOL = "/root/reference/tools/perf_profiling/gen_timeline_json.py"
ROWS = [
    ("Conv_0", "Conv", 0.0, 120.5, 236.027904, 4.1e6, "M=12544 N=64 K=147 tf32 tile=128x64 split=1"),
    ("MaxPool_0", "MaxPool", 120.5, 150.0, 0.0, 4.0e6, ""),
    ("Conv_1, odd name", "Conv", 150.0, 200.0, 25.690112, 1.6e6, "M=3136,N=64"),
    ("Gemm_0", "Gemm", 200.0, 210.0, 4.096, 8.2e6, "split=4"),
]


def _write(path):
    onet.write_timeline_csv(path, ROWS, gpu="NVIDIA B200", gpu_hw_info="148 SMs sm_100", hw_gops=1.1e6, model_name="resnet50")


def test_csv_has_the_reference_columns(tmp_path):
    p = tmp_path / "t.csv"
    _write(p)
    lines = p.read_text().strip().split("\n")
    head = lines[0].split(",")
    assert head[:12] == ["op_name", "op_type", "op_st", "op_ed", "op_computation", "", "cpu", "cpu_hw_info", "gpu", "gpu_hw_info",
                         "hw_computing_power (GOPS)", "model name"]
    assert head[12:] == ["op_bytes", "op_detail"]
    first = lines[1].split(",")
    # what gen_timeline_json.py:41-42 does with the first data row
    hw = first[6:]
    assert float(hw[4]) == 1.1e6 and hw[2] == "NVIDIA B200" and hw[5] == "resnet50"
    assert all(len(ln.split(",")) == 14 for ln in lines)          # commas inside names / details were replaced
    assert lines[3].startswith("Conv_1; odd name,Conv,150.000,200.000,25.690112,")
    with pytest.raises(Exception):
        onet.write_timeline_csv(p, ROWS, hw_gops=0.0)             # the tool divides by it


@pytest.mark.skipif(not os.path.exists(TOOL), reason="reference tree not present")
def test_reference_timeline_tool_reads_the_csv(tmp_path):
    work = tmp_path / "perf"
    (work / "timeline_info").mkdir(parents=True)
    shutil.copy(TOOL, work / "gen_timeline_json.py")             # run from a copy: the tool writes next to its input
    _write(work / "timeline_info" / "resnet50.csv")              # the file name the tool hard-codes
    subprocess.run([sys.executable, "gen_timeline_json.py"], cwd=work, check=True, timeout=60)
    out = json.load(open(work / "timeline_info" / "resnet50.json"))
    assert out["gpu"] == "NVIDIA B200" and out["model_name"] == "resnet50" and out["op_num"] == len(ROWS)
    assert out["total_hardware_computing_power (GOPS)"] == "1100000.000"
    names = [e["name"] for e in out["traceEvents"] if e["ph"] == "X"]
    assert names == ["Conv_0", "MaxPool_0", "Conv_1; odd name", "Gemm_0"]
    total_mflop = sum(r[4] for r in ROWS)
    assert abs(float(out["model_computation (FLOPs(G))"]) - total_mflop * 1e6 / 1024 ** 3) < 1e-3
    assert out["model_eval time"] == "0.210ms"
