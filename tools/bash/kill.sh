#!/usr/bin/env bash
# Forwards to gpt_neox_b200/cluster/kill.sh (reference script: tools/bash/kill.sh).
exec "$(dirname "$0")/../../gpt_neox_b200/cluster/kill.sh" "$@"
