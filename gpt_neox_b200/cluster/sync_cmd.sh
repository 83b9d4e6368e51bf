#!/usr/bin/env bash
# Run a command on every host.  usage: sync_cmd.sh <cmd> [args...]
set -eu
HOSTS="${HOSTS:-/job/hosts}"
echo "Running on all hosts: $*"
pdsh -f 1024 -R ssh -w "^${HOSTS}" "$@"
