"""B200-native configurable hierarchical collectives (allreduce, reduce-scatter, allgather)."""
