#!/usr/bin/env bash
# Run kill.sh on every host of the job.
set -eu
HOSTS="${HOSTS:-/job/hosts}"
HERE="$(cd "$(dirname "$0")" && pwd)"
pdsh -f 1024 -R ssh -w "^${HOSTS}" "bash ${HERE}/kill.sh"
