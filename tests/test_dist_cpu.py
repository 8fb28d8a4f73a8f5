"""Host-side logic of the multi-GPU patterns with world_size-2 gloo ranks on CPU: row / sequence sharding,
weight slicing, and the all-gather assembly of the column-split projection (the projection itself is replaced by the
CPU oracle here; on GPUs it is the librwkvq kernel)."""
import os
import socket

import pytest
import torch


def test_shard_rows_and_sequences():
    import rwkvq_dist as D
    for m in (0, 1, 7, 64, 2049):
        for world in (1, 2, 4, 8):
            spans = [D.shard_rows(m, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == m
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert max(e - s for s, e in spans) - min(e - s for s, e in spans) <= 1
    assert D.shard_sequences(8, 1, 4) == [1, 5]
    assert sorted(sum((D.shard_sequences(9, r, 4) for r in range(4)), [])) == list(range(9))


def test_slice_weight_info_layouts():
    import rwkvq_dist as D
    info = {"weight": torch.arange(512 * 4).reshape(512, 4), "block_scale": torch.arange(512).reshape(512, 1),
            "tensor_scale": torch.tensor(0.5), "qtype": "nvfp4"}
    parts = [D.slice_weight_info(info, r, 2) for r in range(2)]
    assert torch.equal(torch.cat([p["weight"] for p in parts]), info["weight"])
    assert torch.equal(torch.cat([p["block_scale"] for p in parts]), info["block_scale"])
    assert parts[1]["tensor_scale"] is info["tensor_scale"] and parts[0]["qtype"] == "nvfp4"
    with pytest.raises(ValueError):
        D.slice_weight_info(info, 0, 3)
    # a cache derived from the FULL matrix must not travel with a slice; per-input-channel vectors are not sliced even
    # when K happens to equal N; a per-row tensor_scale is
    sq = {"weight": torch.zeros(512, 512), "awq_scale": torch.arange(512.0), "tensor_scale": torch.arange(512.0),
          "block_scale": torch.zeros(512, 32), "block_scale_blocked": torch.zeros(99), "qtype": "nvfp4"}
    p1 = D.slice_weight_info(sq, 1, 2)
    assert "block_scale_blocked" not in p1 and "block_scale_blocked" in sq
    assert p1["awq_scale"].shape == (512,) and torch.equal(p1["tensor_scale"], torch.arange(256.0, 512.0))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_column_split_and_row_sharding_world2():
    """Two gloo ranks as child processes (tests/dist_worker.py); each prints its verdict."""
    import subprocess
    import sys
    port = _free_port()
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "dist_worker.py")
    procs = [subprocess.Popen([sys.executable, worker, str(r), "2", str(port)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r} split=True rows=True" in out, out
