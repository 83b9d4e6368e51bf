#!/usr/bin/env bash
# Forwards to gpt_neox_b200/cluster/multinode_prepare_data.sh (reference script: tools/datasets/multinode_prepare_data.sh).
exec "$(dirname "$0")/../../gpt_neox_b200/cluster/multinode_prepare_data.sh" "$@"
