#!/bin/bash
# Validation loss / perplexity (or lm-evaluation-harness tasks) of a checkpoint, with the model-size blocks of
# run_pretrain.sh (counterpart of examples/linear_moe_qwen2/run_evaluate_mcore_qwen.sh and eval/lm_eval_linear_moe.sh):
#   CKPT=/path/to/checkpoint VALID_DATA=/path/to/valid.json BASE_MODEL=qwen2 MODEL_SIZE=0.5B LA_MODULE=none bash run_evaluate.sh
#   TASKS=piqa,hellaswag TOKENIZER=/path/to/tokenizer ...      runs the harness instead (needs the lm_eval package)
set -e
HERE=$(dirname $0)
GPUS=${GPUS:-1}; EVAL_ITERS=${EVAL_ITERS:-10}; PAD_LEN=${PAD_LEN:-${SEQ_LEN:-2048}}
FLAGS=$(DRY_RUN=1 TRAIN_ITERS=1 GLOBAL_BATCH_SIZE=$(( ${BATCH_SIZE:-4} * GPUS / ${TP:-1} / ${PP:-1} / ${CP:-1} )) bash ${HERE}/run_pretrain.sh)
[ -n "${CKPT}" ] && LOAD="--load ${CKPT} --no-load-optim --no-load-rng" || LOAD=""
[ -n "${VALID_DATA}" ] && DATA="--dataset LLama-Pretrain-Raw --valid-data-path ${VALID_DATA} --train-data-path ${VALID_DATA} --max-padding-length ${PAD_LEN} --eod-mask-loss" || DATA=""
[ -n "${TASKS}" ] && HARNESS="--lm-eval-tasks ${TASKS} --tokenizer-model ${TOKENIZER} --patch-tokenizer-type ${TOKENIZER_TYPE:-Qwen2Tokenizer}" || HARNESS=""
CMD="${HERE}/evaluate.py ${FLAGS} ${LOAD} ${DATA} ${HARNESS} --eval-iters ${EVAL_ITERS} --seed 1234"
if [ -n "${DRY_RUN_EVAL}" ]; then echo ${CMD}; exit 0; fi
torchrun --nnodes 1 --nproc-per-node ${GPUS} --master-addr 127.0.0.1 --master-port ${MASTER_PORT:-29501} ${CMD}
