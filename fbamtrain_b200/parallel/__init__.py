"""Communication and parallelism: NCCL wrapper, rendezvous, peer-memory windows, data parallel
(all-reduce / ZeRO-1 / fused peer-memory kernels), fault-tolerant membership, pipeline and tensor
parallelism."""
