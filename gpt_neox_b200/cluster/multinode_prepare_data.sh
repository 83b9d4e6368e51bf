#!/bin/bash
# Tokenise a corpus with several processes, on one or many nodes.
#
#   srun -N 4 --ntasks-per-node 8 gpt_neox_b200/cluster/multinode_prepare_data.sh files.txt \
#        --tokenizer-type HFTokenizer --vocab-file tokenizer.json --output-prefix data/pile --append-eod
#
# files.txt holds one jsonl path per line. Every process takes a contiguous share of the lines (its rank
# and the number of processes come from RANK / WORLD_SIZE, else from SLURM, else from Open MPI) and writes
# <output-prefix><rank>_<key>_document.{bin,idx}; the parts are merged afterwards with
#   python -m gpt_neox_b200.data.dataset_tools merge --input <dir with the parts> --output-prefix <merged>
# All other arguments are passed on to the preprocessing tool unchanged.
set -euo pipefail
if [[ $# -lt 1 || ! -f "$1" ]]; then
    echo "usage: $0 <file with one input path per line> [preprocess_data arguments...]" >&2
    exit 2
fi
list="$1"
shift
exec python -m gpt_neox_b200.data.preprocess_data --input-list "$list" "$@"
