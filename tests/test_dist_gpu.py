"""Column-split FFN key projection on real GPUs: two NCCL ranks as child processes (tests/dist_gpu_worker.py), the
gather through NCCL and through the library's peer-memory kernels.  Also, on one GPU, the pull that gives up when a
rank never signals (bounded wait, status word, no hang)."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_column_split_ffn_key_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = _free_port()
    worker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "dist_gpu_worker.py")
    procs = [subprocess.Popen([sys.executable, worker, str(r), "2", str(port)], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
             for r in range(2)]
    outs = [p.communicate(timeout=600)[0] for p in procs]
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, "\n".join(l for l in out.splitlines() if "frame #" not in l)[-4000:]
        line = [l for l in out.splitlines() if l.startswith(f"rank {r} ")]
        assert line, out[-3000:]
        verdicts = line[-1].split()[2:]
        assert len(verdicts) == 20 and all(v.endswith("=True/True") for v in verdicts), line[-1]


def test_pull_gives_up_when_a_rank_never_signals():
    """Two 'ranks' emulated by two buffers on one GPU; rank 1 never signals, so rank 0's pull runs into its wait limit,
    records RWKVQ_E_TIMEOUT and returns; after a signal the same pull succeeds."""
    import ctypes
    import rwkvq_abi as abi
    abi.require_device()
    L = abi.lib()
    m, nl = 8, 64
    outs = [torch.zeros((m, 2 * nl), dtype=torch.float16, device="cuda") for _ in range(2)]
    outs[1][:, nl:] = 3.0
    flags = [torch.zeros(8, dtype=torch.int32, device="cuda") for _ in range(2)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    arr = ctypes.c_void_p * 2
    out_arr, flag_arr = arr(*[t.data_ptr() for t in outs]), arr(*[t.data_ptr() for t in flags])
    L.rwkvq_set_wait_limit_us(300)
    try:
        abi.call("rwkvq_allgather_cols_pull", out_arr, flags[0].data_ptr(), 1, 0, 2, m, nl, 2 * nl, status.data_ptr(), abi.stream_ptr())
        torch.cuda.synchronize()
        assert status.item() == abi.E_TIMEOUT and not outs[0].any()
        status.zero_()
        abi.call("rwkvq_peer_signal", flag_arr, 1, 2, 1, abi.stream_ptr())          # "rank 1" delivers epoch 1
        abi.call("rwkvq_allgather_cols_pull", out_arr, flags[0].data_ptr(), 1, 0, 2, m, nl, 2 * nl, status.data_ptr(), abi.stream_ptr())
        torch.cuda.synchronize()
        assert status.item() == 0 and torch.equal(outs[0][:, nl:], outs[1][:, nl:]) and not outs[0][:, :nl].any()
    finally:
        L.rwkvq_set_wait_limit_us(0)
