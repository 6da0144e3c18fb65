#!/bin/bash
# Stop the agents started by start_multi_node.sh. Each agent's process id is read from the pid file the
# launcher wrote on its host; only those process groups are signalled (the reference kills every python
# process by name, multi_node_cmds/stopdown.sh:15-18).
set -euo pipefail
HOSTS=(${HOSTS:?space separated host list})
REPO=${REPO:-$(cd "$(dirname "$0")/.." && pwd)}
for h in "${HOSTS[@]}"; do
  ssh "$h" "cd $REPO && for f in torchrun_*.pid; do [ -f \$f ] && kill -- -\$(cat \$f) 2>/dev/null; rm -f \$f; done" &
done
wait
