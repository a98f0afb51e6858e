"""bind_host_to_device is best effort: without a GPU (or on a platform that exposes no NUMA
information) it changes nothing and says so."""
import os


def test_bind_without_gpu_is_a_no_op():
    from hbq_b200.shard import bind_host_to_device
    before = os.sched_getaffinity(0)
    info = bind_host_to_device(0)
    assert set(info) == {"numa_node", "cpus_bound", "mempolicy"}
    if info["numa_node"] is None:
        assert info["cpus_bound"] == 0 and info["mempolicy"] is False
        assert os.sched_getaffinity(0) == before
