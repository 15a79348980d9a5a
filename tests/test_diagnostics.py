"""The stage-dump file format and the decode trace, without a GPU."""
import json
import struct

import numpy as np
import pytest
import torch

from mimirmind_b200.engine.diagnostics import DecodeTrace, StageDump, read_stage_dump


def test_stage_dump_file_is_three_uint32_and_float32_rows(tmp_path):
    d = StageDump(str(tmp_path / "p"))
    rows = torch.arange(6, dtype=torch.float32).reshape(2, 3) * 0.5
    d.write(4, "attn_out", rows.to(torch.bfloat16))                 # any float dtype is written as float32
    d.write(0, "Qcur", torch.ones(5, 2, 4))                         # more than two dimensions: rows x the rest
    raw = (tmp_path / "p-blk4-attn_out.bin").read_bytes()
    assert struct.unpack("<III", raw[:12]) == (4, 2, 3) and len(raw) == 12 + 6 * 4
    assert np.array_equal(np.frombuffer(raw[12:], dtype="<f4"), rows.numpy().ravel())
    block, back = read_stage_dump(str(tmp_path / "p-blk0-Qcur.bin"))
    assert block == 0 and back.shape == (5, 8) and (back == 1).all()
    assert d.files_written == 2
    (tmp_path / "bad.bin").write_bytes(struct.pack("<III", 0, 2, 2) + b"\x00" * 8)
    with pytest.raises(ValueError, match="header says 2 x 2"):
        read_stage_dump(str(tmp_path / "bad.bin"))


def test_decode_trace_lines(tmp_path):
    t = DecodeTrace(str(tmp_path / "t.ndjson"))
    t.step(8, 3.21987)
    t.step(7, 3.1)
    t.close()
    lines = [json.loads(l) for l in open(tmp_path / "t.ndjson")]
    assert [l["step"] for l in lines] == [0, 1] and lines[0]["tokens"] == 8 and lines[0]["wall_ms"] == 3.22
    assert set(lines[1]) == {"step", "tokens", "wall_ms", "sm_mhz", "gpu_c"}
