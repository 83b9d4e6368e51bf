#!/usr/bin/env bash
# Copy a directory tree to the same absolute path on every host.  usage: syncdir.sh <dir>
set -eu
HOSTS="${HOSTS:-/job/hosts}"
d="$(realpath "$1")"
echo "Syncing directory $d"
pdcp -f 1024 -R ssh -w "^${HOSTS}" -r "$d" "$(dirname "$d")"
