#!/usr/bin/env bash
# Forwards to gpt_neox_b200/cluster/killall.sh (reference script: tools/bash/killall.sh).
exec "$(dirname "$0")/../../gpt_neox_b200/cluster/killall.sh" "$@"
