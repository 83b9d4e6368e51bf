#!/usr/bin/env bash
# Copy one file to the same absolute path on every host.  usage: sync.sh <file>
set -eu
HOSTS="${HOSTS:-/job/hosts}"
f="$(realpath "$1")"
echo "Syncing $f"
pdcp -f 1024 -R ssh -w "^${HOSTS}" "$f" "$f"
