"""B200-native MoE all-to-all dispatch / expert placeholder / combine.

Public surface (mirrors the reference task, amd-distributed/all2all):

* ``MoEConfig``, ``RankTestData``, ``generate_input`` -- the task contract
  (reference.py:10-51, :237-253).
* ``custom_kernel(data)`` -- the plugin entry point (task.py:8-9); runs the
  hand-written sm_100a kernels through the C-ABI library ``liba2a.so``.
* ``check_implementation(data, output, reference_output)`` -- the task's checker
  (reference.py:275-283) for harnesses; import it from ``.all2all``.
* ``A2AContext`` -- per-process-group state: symmetric receive buffers, peer
  mappings, flags (the role ``P2PState`` plays in submission_v9.py:880-947).

Importing this package does not load the CUDA library; the first use of
``A2AContext`` / ``custom_kernel`` does, and raises if it is missing.
"""
from .task import (  # noqa: F401
    MoEConfig,
    RankTestData,
    generate_input,
    workload_input,
    reference_task_input,
    WORKLOADS,
    REFERENCE_TESTS,
    REFERENCE_BENCHMARKS,
    input_t,
    output_t,
)
