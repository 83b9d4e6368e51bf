"""Checkpoint IO in the Megatron/DeepSpeed on-disk layout."""
