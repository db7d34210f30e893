"""Planner cost-model constants (profiler.py of the reference): shapes on the CPU, measurement on a GPU."""
import pytest
import torch


def test_case_lengths_follow_the_reference_shapes():
    from hap_b200 import profiler
    total, lengths, rows = profiler.case_lengths("all_gather", 4 << 20, 8, 1.0)
    assert total == 4096 and lengths == [512] * 8 and rows == [32] * 8
    total, lengths, rows = profiler.case_lengths("all_to_all", 16 << 20, 4, 3.0)       # [3,1,1,1] / 6
    assert total == 16384 and sum(lengths) == total and lengths[0] == 8192 and sum(rows) == 256 and rows[0] == 128
    cfg = profiler.planner_config({op + "_bandwidth": 10 + i for i, op in enumerate(profiler.OPS)}, [1.5e12, 2e12])
    assert cfg["device_flops"] == [1500000000000, 2000000000000]
    assert set(cfg) == {"device_flops"} | {op + "_bandwidth" for op in profiler.OPS}


@pytest.mark.gpu
def test_bandwidths_on_two_virtual_ranks():
    import hap_b200
    from hap_b200 import profiler
    dev = torch.device("cuda:0")
    comm = hap_b200.local_comm(2, dev, stage_bytes=8 << 20, heap_bytes=48 << 20)
    try:
        bw = profiler.measure_bandwidths(comm, skewness=2.0, sizes=(1 << 20, 4 << 20), reps=3, warmup=2)
        assert set(bw) == {op + "_bandwidth" for op in profiler.OPS}
        assert all(v > 1e9 for v in bw.values()), bw          # anything on one B200 moves more than 1 GB/s
        comm.check()
        w = torch.randn(1024, 1024, device=dev, dtype=torch.bfloat16)
        flops = profiler.measure_device_flops(lambda: hap_b200.linear(w, w), 2 * 1024 ** 3, warmup=3, reps=3)
        assert flops > 1e12
    finally:
        comm.destroy()
