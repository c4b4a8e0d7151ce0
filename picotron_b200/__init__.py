"""picotron_b200: a Blackwell-native 4D-parallel (DP x PP x CP x TP) Llama pre-training framework.

Layout of the package:

* ``process_group_manager`` -- the dp x pp x cp x tp rank grid and its process groups.
* ``config``                -- typed view of the JSON experiment file plus offline model presets.
* ``models``                -- the Llama decoder built from fused ops with hand-derived backward passes.
* ``ops``                   -- every hot op: a CUDA (sm_100a) kernel and a plain PyTorch restatement
                               that is used on CPU/Gloo and as the oracle in the tests.
* ``parallel``              -- tensor / pipeline / context / data parallel strategies.
* ``comm``                  -- symmetric-memory runtime and the fused compute+collective kernels.
* ``optim``                 -- multi-tensor AdamW over fp32 gradient buckets (optionally sharded over the replicas),
                               learning-rate schedule, global-norm clipping.
* ``trainer``               -- start-up sequence and the optimizer step; evaluation, replica and non-finite checks.
* ``checkpoint``, ``reshard`` -- per-(tp, pp)-rank checkpoints, Hugging Face import/export, re-cutting for another grid.
* ``data``, ``generate``, ``utils`` -- input pipeline, greedy decoding for a quick look at a checkpoint, logging,
                               metrics, tracing, watchdog and the memory planner.
"""

__version__ = "0.1.0"
