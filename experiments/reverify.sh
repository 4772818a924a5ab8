#!/bin/bash
# Re-run the throughput / loss table and, optionally, compare it with a trusted earlier run.
# Use it before committing a change that could touch training numerics or speed (kernels, optimizer, planner).
#
#   bash experiments/reverify.sh                               # default rows, writes runs/reverify_<UTC time>/
#   bash experiments/reverify.sh --baseline runs/reverify_X    # + diff: loss equal to 4 decimals, tok/s within 5 %
#   bash experiments/reverify.sh --include-gemma --include-moe # more rows
#   bash experiments/reverify.sh --gpus 8 --out runs/my_rerun  # one torch.distributed.run job per row
#
# Environment: PY (python to use, default python), FLEXTRAIN_VERIFIED_ROWS (comma list of <dims name>:<mode>,
# replaces the default rows).  Exit status: 0 when every row ran (and, with --baseline, every row matched).
set -euo pipefail
ROOT="$(cd "$(dirname "${BASH_SOURCE[0]}")/.." && pwd)"
PY="${PY:-python}"
ROWS="${FLEXTRAIN_VERIFIED_ROWS:-llama3_2_1B:full,llama3_1_8B:full,llama3_1_8B:lora,qwen3_8B:full}"
OUT=""; BASELINE=""; GPUS=1; EXTRA=()
while [[ $# -gt 0 ]]; do
  case "$1" in
    --include-gemma) ROWS="$ROWS,gemma2_2B:full,gemma3_4B:full"; shift ;;
    --include-moe)   ROWS="$ROWS,qwen3_30B_A3B:lora,olmoe_1B_7B:full"; shift ;;
    --baseline)      BASELINE="$2"; shift 2 ;;
    --out)           OUT="$2"; shift 2 ;;
    --gpus)          GPUS="$2"; shift 2 ;;
    *)               EXTRA+=("$1"); shift ;;
  esac
done
OUT="${OUT:-$ROOT/runs/reverify_$(date -u +%Y%m%dT%H%M%SZ)}"
ARGS=(--rows "$ROWS" --gpus "$GPUS" --out "$OUT")
[[ -n "$BASELINE" ]] && ARGS+=(--baseline "$BASELINE")
echo "[reverify] rows: $ROWS"
echo "[reverify] out:  $OUT"
"$PY" "$ROOT/experiments/verified_runs.py" "${ARGS[@]}" "${EXTRA[@]}"
echo "[reverify] table: $OUT/table.md"
