#!/usr/bin/env bash
# End the training ranks that the launcher started on THIS host (exact PIDs from its pid file).
set -u
PIDFILE="${NEOX_PIDFILE:-/tmp/gpt_neox_b200.$(id -u).pids}"
[ -f "$PIDFILE" ] || { echo "no pid file at $PIDFILE: nothing to do"; exit 0; }
while read -r pid; do
  [ -n "$pid" ] && kill -TERM "$pid" 2>/dev/null && echo "sent TERM to $pid"
done < "$PIDFILE"
sleep 2
while read -r pid; do
  [ -n "$pid" ] && kill -0 "$pid" 2>/dev/null && kill -KILL "$pid" 2>/dev/null && echo "sent KILL to $pid"
done < "$PIDFILE"
rm -f "$PIDFILE"
