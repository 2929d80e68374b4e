"""B200-native communication runtime with the capabilities of DLSlime.

Sub-packages: ``ops`` (sm_100a kernels), ``parallel`` (symmetric memory and
process-group plumbing), ``models`` (the MoE layer and KV-transfer workloads),
``peer_agent`` / ``nanoctrl`` / ``rpc`` / ``cache`` (control plane and services).
"""

__version__ = "0.1.0"
