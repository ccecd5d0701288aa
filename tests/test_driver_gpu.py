"""The bench driver end to end on the GPU: commands file -> CSV with one row per command."""

import csv
import shlex

import pytest

from iree_turbine_b200 import driver

pytestmark = pytest.mark.gpu


def test_commands_file_round_trip(tmp_path):
    commands = [
        "gemmfp16 --a_w 256 --a_h 512 --b_w 384 --transB 1 --iter 5",
        "gemmfp16 --a_w 256 --a_h 512 --b_w 384 --iter 5",
        "gemm --a_w 64 --a_h 64 --b_w 64 --iter 3",
        "aten::mm \"[[256, 512], [512, 128]]\" \"['c10::BFloat16', 'c10::BFloat16']\" \"[[512, 1], [1, 512]]\" \"['', '']\" --iter 4",
        "aten::scaled_dot_product_attention \"[[2, 8, 256, 128], [2, 8, 256, 128], [2, 8, 256, 128], [], [], [], [], []]\" "
        "\"['c10::Half', 'c10::Half', 'c10::Half', '', 'Scalar', 'Scalar', 'Scalar', 'Scalar']\" "
        "\"[[262144, 32768, 128, 1], [262144, 32768, 128, 1], [262144, 32768, 128, 1], [], [], [], [], []]\" "
        "\"['', '', '', 'None', '0.0', 'True', 'None', 'False']\" --iter 4",
    ]
    cf = tmp_path / "commands.txt"
    cf.write_text("# comment\n" + "\n".join(commands) + "\n")
    out = tmp_path / "stats.csv"
    assert driver.main([f"--csv={out}", "--backends=b200k", "--backends=torch", f"--commands-file={cf}"]) == 0
    rows = list(csv.DictReader(out.read_text().splitlines()))
    assert [r["arguments"] for r in rows] == [shlex.join(shlex.split(c)) for c in commands]
    assert rows[0]["b200k num_dispatches"] == "5" and float(rows[0]["b200k min"]) > 0
    assert rows[1]["b200k num_dispatches"] == "5"          # B stored [K, N]: read as it is
    assert rows[2]["b200k min"] == "N.A." and rows[2]["torch num_dispatches"] == "3"   # float32: torch only
    assert rows[3]["b200k num_dispatches"] == "4" and rows[4]["b200k num_dispatches"] == "4"
    for r in rows:
        assert float(r["torch min"]) <= float(r["torch mean"]) <= float(r["torch max"])
