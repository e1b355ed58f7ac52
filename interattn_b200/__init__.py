"""interattn_b200: B200 (sm_100a) kernels for condition-block sparse decode attention.

Public surface:

* ``interattn_b200.ops``            - batched / paged operators over the C ABI
* ``interattn_b200.reference_api``  - the reference project's operator names and
  signatures (``_build_prompt_blocks``, ``_select_prompt_blocks``,
  ``_run_condition_block_selection_stats``,
  ``_condition_block_decode_output_fused_triton``, the Hugging Face attention hook)
* ``interattn_b200.partition``      - 1/2/4/8-GPU sharding of the step
* ``interattn_b200.build``          - in-tree nvcc build of the shared library

Importing the package does not load the CUDA library; the first operator call
does, and raises if it is missing.
"""

__version__ = "0.1.0"
