#!/usr/bin/env bash
# Forwards to gpt_neox_b200/cluster/sync.sh (reference script: tools/bash/sync.sh).
exec "$(dirname "$0")/../../gpt_neox_b200/cluster/sync.sh" "$@"
