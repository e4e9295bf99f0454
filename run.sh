#!/usr/bin/env bash
# One-click demo: build the kernel library, (optionally) search a schedule, train a few
# iterations of the 8-layer Llama-70B-shaped model with tensor + sequence parallelism.
# Settings are the variables below; every flag is the Megatron-style flag of train.py.
set -euo pipefail
cd "$(dirname "$0")"

GPUS=${GPUS:-8}                    # GPUs of this node = tensor-parallel size x context x pipeline x data
TP=${TP:-$GPUS}
CP=${CP:-1}
PP=${PP:-1}
MODEL=${MODEL:-llama}              # llama | gpt
LAYERS=${LAYERS:-8}
HIDDEN=${HIDDEN:-8192}
FFN=${FFN:-28672}
HEADS=${HEADS:-64}
KV_HEADS=${KV_HEADS:-8}
SEQ=${SEQ:-4096}
VOCAB=${VOCAB:-128256}
GLOBAL_BATCH=${GLOBAL_BATCH:-32}
MICRO_BATCH=${MICRO_BATCH:-4}
ITERS=${ITERS:-5}
DHELLAM=${DHELLAM:-true}           # false = one strand, no forward/backward pairing
SEARCH=${SEARCH:-false}            # true = profile the ops on this machine and search a schedule first
SCHEDULE=${SCHEDULE:-}             # strategy file; empty = built-in schedule (or the searched one)
DATA=${DATA:-}                     # flat token file "<path>[:dtype]"; empty = synthetic tokens
PORT=${PORT:-29511}

python -m dhellam_b200.kernels.build

LAUNCH=(python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port "$PORT")
MODEL_ARGS=(--num-layers "$LAYERS" --hidden-size "$HIDDEN" --num-attention-heads "$HEADS" --seq-length "$SEQ"
            --max-position-embeddings "$SEQ" --vocab-size "$VOCAB" --disable-bias-linear --untie-embeddings-and-output-weights)
if [ "$MODEL" = llama ]; then
  MODEL_ARGS+=(--ffn-hidden-size "$FFN" --swiglu --normalization RMSNorm --group-query-attention --num-query-groups "$KV_HEADS"
               --position-embedding-type rope)
elif [ "$MODEL" = gpt ]; then
  MODEL_ARGS+=(--normalization LayerNorm --position-embedding-type learned_absolute)
else
  echo "unsupported model type: $MODEL" >&2; exit 1
fi
PARALLEL_ARGS=(--tensor-model-parallel-size "$TP" --context-parallel-size "$CP" --pipeline-model-parallel-size "$PP" --sequence-parallel)

if [ "$SEARCH" = true ]; then
  "${LAUNCH[@]}" -m dhellam_b200.search.run "${MODEL_ARGS[@]}" "${PARALLEL_ARGS[@]}" --micro-batch-size "$MICRO_BATCH" --search-dir search_out
  SCHEDULE=search_out/config/best.json
fi

TRAIN_ARGS=(--global-batch-size "$GLOBAL_BATCH" --micro-batch-size "$MICRO_BATCH" --train-iters "$ITERS" --bf16
            --weight-decay 0.1 --adam-beta1 0.9 --adam-beta2 0.95 --init-method-std 0.006 --clip-grad 1.0
            --lr 6.0e-5 --min-lr 6.0e-6 --lr-decay-style cosine --lr-warmup-fraction .001 --lr-decay-iters 430000
            --log-interval 1 --log-throughput)
[ "$DHELLAM" = true ] && TRAIN_ARGS+=(--dhellam)
[ -n "$SCHEDULE" ] && TRAIN_ARGS+=(--schedule-config "$SCHEDULE")
[ -n "$DATA" ] && TRAIN_ARGS+=(--data-path "$DATA")

exec "${LAUNCH[@]}" train.py "${MODEL_ARGS[@]}" "${PARALLEL_ARGS[@]}" "${TRAIN_ARGS[@]}"
