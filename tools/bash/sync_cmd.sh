#!/usr/bin/env bash
# Forwards to gpt_neox_b200/cluster/sync_cmd.sh (reference script: tools/bash/sync_cmd.sh).
exec "$(dirname "$0")/../../gpt_neox_b200/cluster/sync_cmd.sh" "$@"
