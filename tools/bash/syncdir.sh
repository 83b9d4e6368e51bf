#!/usr/bin/env bash
# Forwards to gpt_neox_b200/cluster/syncdir.sh (reference script: tools/bash/syncdir.sh).
exec "$(dirname "$0")/../../gpt_neox_b200/cluster/syncdir.sh" "$@"
