"""CPU: host-side helpers of the host-buffer pipeline that need no device."""
import os

from fast_polynomial_transcendentals_b200 import pipeline


def test_numa_binding_is_a_no_op_without_a_device():
    before = os.sched_getaffinity(0)
    assert pipeline.bind_host_thread_to_device_node(0) is None or os.sched_getaffinity(0) <= before
    import torch
    if not torch.cuda.is_available():
        assert os.sched_getaffinity(0) == before
