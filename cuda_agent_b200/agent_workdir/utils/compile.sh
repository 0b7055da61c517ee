#!/bin/bash
# Timed wrapper around `python3 -m utils.compile` (run from the workspace
# directory); prints "[TIME] Compilation took Ns" and passes the exit status on,
# like the reference's utils/compile.sh:3-12. Arguments go to utils.compile.
t0=$(date +%s.%N)
python3 -m utils.compile "$@"
status=$?
t1=$(date +%s.%N)
printf '[TIME] Compilation took %.2fs\n' "$(echo "$t1 - $t0" | bc -l 2>/dev/null || awk "BEGIN{print $t1-$t0}")"
exit $status
