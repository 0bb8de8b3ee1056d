#!/bin/sh
# Row-sharded training on all GPUs of a node: the entity table, its gradients and optimiser moments are split by rows
# across the GPUs and the kernels exchange rows and gradients over NVLink themselves.
#   KvsAll family:   sh examples/sharded_training.sh KGs/FB15k-237 ComplEx KvsAll
#   sampled family:  sh examples/sharded_training.sh KGs/FB15k-237 TransE NegSample --neg_ratio 64
DATA=${1:?dataset dir}; MODEL=${2:-ComplEx}; ST=${3:-KvsAll}; shift 3 2>/dev/null
exec python -m torch.distributed.run --standalone --local-addr 127.0.0.1 --nproc_per_node=gpu -m dice_embeddings_b200 \
    --dataset_dir "$DATA" --model "$MODEL" --scoring_technique "$ST" --trainer Sharded --embedding_dim 256 \
    --batch_size 4096 --num_epochs 100 --lr 0.1 --path_to_store_single_run "Experiments/sharded_${MODEL}_${ST}" "$@"
