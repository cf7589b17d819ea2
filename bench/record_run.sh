#!/bin/bash
# End-to-end record-style run on N GPUs of one node, through the command-line entry points only:
#   synthetic dataset -> training in `record` mode to a wall-clock cap (EMA, SWA, late QAT as the schedule reaches them)
#   -> pre-quantisation diagnostic -> GPTQ int6 export with self-generated calibration -> score-first TTT evaluation of the
#   round-tripped artifact (all inside the trainer) -> sliding-window evaluation of the same artifact with the eval CLI.
# Counterpart of the reference's 10-minute record script (records/track_10min_16mb/2026-03-23_LeakyReLU_LegalTTT_ParallelMuon/
# train_gpt.py:1643-1765 and its log train_seed1337.log:66-77,274).
#
#   bench/record_run.sh <gpus> <wallclock cap in seconds> <work dir> [validation tokens] [training tokens]
set -e
N=${1:-8}; CAP=${2:-150}; DIR=${3:-/tmp/pgb_record}; VAL=${4:-8519681}; TRAIN=${5:-134217728}
HERE="$(cd "$(dirname "$0")/.." && pwd)"
cd "$HERE"
python -m parameter_golf_b200.data.shards --root "$DIR/data" --vocab 1024 --train-tokens "$TRAIN" --val-tokens "$VAL" --train-shards 2
LAUNCH="python -m torch.distributed.run --nnodes=1 --nproc-per-node $N --master-addr 127.0.0.1"
$LAUNCH --master-port 29811 -m parameter_golf_b200.train run --spec specs/record_profile.toml --mode record \
    allow_unsupported_variants=true train.world_size=$N train.max_wallclock_seconds=$CAP train.train_log_every=100 \
    "train.train_data_pattern=$DIR/data/fineweb_train_*.bin" "train.validation_data_pattern=$DIR/data/fineweb_val_*.bin" \
    "train.artifact_path=$DIR/artifact.pgrs"
$LAUNCH --master-port 29812 -m parameter_golf_b200.evalcli --artifact "$DIR/artifact.pgrs" --spec specs/record_profile.toml \
    --val-pattern "$DIR/data/fineweb_val_*.bin" --bytes seeded --device cuda eval.adaptation_backend=none
