"""Host-side distributed services: KV-cache event publishing, the NCCL ctypes binding, stateless
process groups, KV offload tiers and expert load balancing."""
