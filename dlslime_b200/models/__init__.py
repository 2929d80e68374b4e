"""What is built from the operators: the expert-parallel MoE layer and the prefill -> decode KV transfer.

Import the submodules (``dlslime_b200.models.moe``, ``dlslime_b200.models.pd_kv``); they need CUDA.
"""
