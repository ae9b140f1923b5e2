#!/bin/bash
# Launcher with the reference's switch blocks (examples/linear_moe_qwen2/run_pretrain_qwen.sh:17-62,126-365):
#   MODEL_SIZE  qwen2: 0.5B 0.5Boriginal 1.5B 7B 72B A0.3B A1B A14B | llama3: 0.3B 1B 8B | mixtral: Small 8x7B | deepseek_v2: A2.4B A21B
#   LA_MODULE   any --la-module value or "none" (pure softmax attention); LAYER_TYPE_LIST  L/N pattern (M/*/- for mamba2)
#   PR fp16|bf16|fp8, AC full|sel|none, DO true|false, SP true|false, TP PP CP EP sizes
set -e
BASE_MODEL=${BASE_MODEL:-qwen2}; MODEL_SIZE=${MODEL_SIZE:-A0.3B}; LA_MODULE=${LA_MODULE:-gla}
LAYER_TYPE_LIST=${LAYER_TYPE_LIST:-LLLLLLLLLLLL}; GPUS=${GPUS:-8}
TP=${TP:-1}; PP=${PP:-1}; CP=${CP:-1}; EP=${EP:-1}; SP=${SP:-false}; DO=${DO:-true}; AC=${AC:-sel}; PR=${PR:-bf16}
BATCH_SIZE=${BATCH_SIZE:-4}; GLOBAL_BATCH_SIZE=${GLOBAL_BATCH_SIZE:-64}; SEQ_LEN=${SEQ_LEN:-2048}
LR=${LR:-1e-4}; MIN_LR=${MIN_LR:-1e-5}; TRAIN_ITERS=${TRAIN_ITERS:-1000}; WARMUP=${WARMUP:-100}
DATASET=${DATASET:-Synthetic}; DATA_PATH=${DATA_PATH:-}; OUT=${OUT:-./output}
case "${BASE_MODEL}-${MODEL_SIZE}" in
  qwen2-0.5B)  M="--num-layers 24 --hidden-size 512 --num-attention-heads 16 --ffn-hidden-size 4864 --rotary-base 1000000 --extra-vocab-size 293";;
  qwen2-0.5Boriginal) M="--num-layers 24 --hidden-size 896 --num-attention-heads 14 --group-query-attention --num-query-groups 2 --ffn-hidden-size 4864 --rotary-base 1000000 --extra-vocab-size 293";;
  qwen2-72B)   M="--num-layers 80 --hidden-size 8192 --num-attention-heads 64 --group-query-attention --num-query-groups 8 --ffn-hidden-size 29568 --rotary-base 1000000 --extra-vocab-size 421";;
  qwen2-1.5B)  M="--num-layers 28 --hidden-size 1536 --num-attention-heads 12 --group-query-attention --num-query-groups 2 --ffn-hidden-size 8960 --rotary-base 1000000 --extra-vocab-size 293";;
  qwen2-7B)    M="--num-layers 28 --hidden-size 3584 --num-attention-heads 28 --group-query-attention --num-query-groups 4 --ffn-hidden-size 18944 --rotary-base 1000000 --extra-vocab-size 421";;
  qwen2-A0.3B) M="--num-layers 12 --hidden-size 1024 --num-attention-heads 8 --ffn-hidden-size 896 --num-experts 64 --moe-router-topk 8 --moe-ffn-hidden-size 896 --rotary-base 10000 --extra-vocab-size 293";;
  qwen2-A1B)   M="--num-layers 16 --hidden-size 2048 --num-attention-heads 16 --ffn-hidden-size 1024 --num-experts 64 --moe-router-topk 8 --moe-ffn-hidden-size 1024 --extra-vocab-size 293";;
  qwen2-A14B)  M="--num-layers 28 --hidden-size 3584 --num-attention-heads 28 --group-query-attention --num-query-groups 4 --ffn-hidden-size 18944 --num-experts 64 --moe-router-topk 8 --moe-ffn-hidden-size 2560 --shared-moe-ffn-hidden-size 20480 --enable-shared-expert --rotary-base 1000000 --extra-vocab-size 293";;
  llama3-0.3B) M="--num-layers 12 --hidden-size 1024 --num-attention-heads 32 --group-query-attention --num-query-groups 8 --ffn-hidden-size 4096 --rotary-base 500000 --norm-epsilon 1e-5 --extra-vocab-size 256";;
  llama3-1B)   M="--num-layers 16 --hidden-size 2048 --num-attention-heads 32 --group-query-attention --num-query-groups 8 --ffn-hidden-size 8192 --rotary-base 500000 --norm-epsilon 1e-5 --extra-vocab-size 256";;
  llama3-8B)   M="--num-layers 32 --hidden-size 4096 --num-attention-heads 32 --group-query-attention --num-query-groups 8 --ffn-hidden-size 14336 --rotary-base 500000 --norm-epsilon 1e-5 --extra-vocab-size 256";;
  mixtral-Small) M="--num-layers 8 --hidden-size 1024 --num-attention-heads 8 --ffn-hidden-size 14336 --num-experts 8 --moe-router-topk 2 --moe-aux-loss-coeff 1e-2 --init-method-std 0.006";;
  mixtral-8x7B)  M="--num-layers 32 --hidden-size 4096 --num-attention-heads 32 --group-query-attention --num-query-groups 8 --ffn-hidden-size 14336 --num-experts 8 --moe-router-topk 2 --moe-aux-loss-coeff 1e-2 --init-method-std 0.006";;
  deepseek_v2-A2.4B) M="--num-layers 27 --hidden-size 2048 --num-attention-heads 16 --ffn-hidden-size 10944 --num-experts 64 --moe-router-topk 6 --moe-ffn-hidden-size 1408 --enable-shared-expert --num-shared-experts 2 --shared-moe-ffn-hidden-size 2816 --moe-layer-freq 1 --kv-lora-rank 512 --qk-nope-head-dim 128 --qk-rope-head-dim 64 --v-head-dim 128 --rotary-scaling-factor 40 --extra-vocab-size 2400";;
  deepseek_v2-A21B)  M="--num-layers 60 --hidden-size 5120 --num-attention-heads 128 --ffn-hidden-size 12288 --num-experts 160 --moe-router-topk 6 --moe-ffn-hidden-size 1536 --enable-shared-expert --num-shared-experts 2 --shared-moe-ffn-hidden-size 3072 --q-lora-rank 1536 --moe-layer-freq 1 --kv-lora-rank 512 --extra-vocab-size 2400";;
  *) echo "unknown ${BASE_MODEL}-${MODEL_SIZE}"; exit 1;;
esac
# per-family switches of the reference launchers (run_pretrain_qwen.sh:430-445, run_pretrain_mcore_llama.sh:321-332,
# run_pretrain_mistral.sh:313-322, run_pretrain_deepseek.sh:349-361): tokenizer vocabulary, QKV bias, norm kind and epsilon
case "${BASE_MODEL}" in
  qwen2)       F="--add-qkv-bias --normalization RMSNorm --norm-epsilon 1e-6 --vocab-size 151643";;
  llama3)      F="--normalization RMSNorm --vocab-size 128000";;
  mixtral)     F="--normalization LayerNorm --vocab-size 32000 --moe-router-load-balancing-type aux_loss";;
  deepseek_v2) F="--normalization RMSNorm --norm-epsilon 1e-6 --rotary-base 10000 --vocab-size 100000 --moe-router-load-balancing-type aux_loss";;
esac
[ "$LA_MODULE" = "none" ] && LA="" || LA="--use-la-module --la-module ${LA_MODULE} --la-mode chunk --la-output-norm rmsnorm --la-gate-fn swish"
if [ "$LA_MODULE" = "mamba2" ]; then LA="$LA --hybrid-override-pattern ${LAYER_TYPE_LIST}"; elif [ -n "$LA" ]; then LA="$LA --layer-type-list ${LAYER_TYPE_LIST}"; fi
[ "$PR" = "fp16" ] && P="--fp16"; [ "$PR" = "bf16" ] && P="--bf16"; [ "$PR" = "fp8" ] && P="--bf16 --fp8-hybrid --fp8-amax-history-len 1024 --fp8-amax-compute-algo max"
[ "$AC" = "full" ] && A="--recompute-granularity full --recompute-method uniform"; [ "$AC" = "sel" ] && A="--recompute-activations"; [ "$AC" = "none" ] && A=""
[ "$DO" = "true" ] && D="--use-distributed-optimizer" || D=""
[ "$SP" = "true" ] && S="--sequence-parallel" || S=""
[ -n "$DATA_PATH" ] && DP="--data-path ${DATA_PATH}" || DP=""
ARGS="--base-model ${BASE_MODEL} ${M} ${F} ${LA} ${P} ${A} ${D} ${S} ${DP} \
  --save ${OUT}/checkpoint --split 99,1,0 --lr ${LR} --min-lr ${MIN_LR} --lr-decay-style cosine --weight-decay 0.1 \
  --adam-beta1 0.9 --adam-beta2 0.95 --clip-grad 1.0 --init-method-std 0.008 --attention-dropout 0.0 --hidden-dropout 0.0 \
  --lr-decay-iters ${TRAIN_ITERS} --lr-warmup-iters ${WARMUP} --train-iters ${TRAIN_ITERS} \
  --micro-batch-size ${BATCH_SIZE} --global-batch-size ${GLOBAL_BATCH_SIZE} --seq-length ${SEQ_LEN} \
  --max-position-embeddings ${SEQ_LEN} --log-interval 10 --eval-interval 100000 --eval-iters 10 --save-interval 1000 \
  --tensorboard-dir ${OUT}/tensorboard --tensor-model-parallel-size ${TP} --pipeline-model-parallel-size ${PP} \
  --context-parallel-size ${CP} --expert-model-parallel-size ${EP} --dataset ${DATASET} --swiglu \
  --use-rotary-position-embeddings --position-embedding-type rope --untie-embeddings-and-output-weights \
  --disable-bias-linear --rotary-percent 1.0"
if [ -n "${DRY_RUN}" ]; then echo ${ARGS}; exit 0; fi      # print the training flags only (used by the tests)
mkdir -p ${OUT}/log ${OUT}/checkpoint
torchrun --nnodes 1 --nproc-per-node ${GPUS} --master-addr 127.0.0.1 --master-port ${MASTER_PORT:-29500} \
  $(dirname $0)/pretrain.py ${ARGS} 2>&1 | tee ${OUT}/log/$(date +%Y.%m.%d-%H.%M.%S).log
