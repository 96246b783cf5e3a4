#!/usr/bin/env bash
# The whole artifact flow on one node, phase by phase: profile the partitions, compose and plan, train with every
# method, compare energy and time.  Counterpart of the reference's tests/artifact scripts (kareus_run_bayesian.sh,
# megatron_perseus_run_profiling.sh, run_megatron.sh, run_nanobatch.sh, run_perseus.sh, run_kareus.sh,
# compare_method.py).  Everything is a `python -m kareus_b200.cli.<driver>` call under torchrun; edit freely.
#
#   NPROC=8 TP=8 MODEL=llama3.2_3b bash examples/artifact_flow.sh            # B200 node
#   NPROC=2 TP=2 MODEL=tiny SEQ=32 MBS=4 GBS=8 STEPS=4 QUICK=1 bash examples/artifact_flow.sh   # CPU smoke run
#
# Clock mode: "advisory" (default) leaves the GPU clocks alone and profiles at the default clock; "locked" sets them
# through NVML and needs the rights to do so.
set -euo pipefail

MODEL=${MODEL:-llama3.2_3b}; NPROC=${NPROC:-8}; TP=${TP:-$NPROC}; PP=${PP:-1}; CP=${CP:-1}
MBS=${MBS:-8}; GBS=${GBS:-64}; SEQ=${SEQ:-4096}; STEPS=${STEPS:-30}
WORK=${WORK:-kareus_runs}; GPU_TYPE=${GPU_TYPE:-B200}; CLOCK_MODE=${CLOCK_MODE:-advisory}
TP_COMM=${TP_COMM:-sp_fused}; MASTER_PORT=${MASTER_PORT:-6000}; QUICK=${QUICK:-0}
SKIP_PROFILING=${SKIP_PROFILING:-false}; FRONTIER=${FRONTIER:-false}
PERSEUS_METHODS=${PERSEUS_METHODS:-"perseus nanobatch_perseus"}      # frequency-only plans: one / two nanobatches
# with context parallelism the partition plan covers the all-reduce flavour of tensor parallelism
[ "$CP" -gt 1 ] && TP_COMM=allreduce
TAG="cp${CP}_tp${TP}_mbs${MBS}_seq${SEQ}"
RUN="python -m torch.distributed.run --nnodes=1 --nproc-per-node ${NPROC} --master-addr 127.0.0.1 --master-port ${MASTER_PORT}"
# the partition profiler works on one pipeline stage: the ranks of one tensor x context parallel group
NPROF=$((TP * CP))
RUNP="python -m torch.distributed.run --nnodes=1 --nproc-per-node ${NPROF} --master-addr 127.0.0.1 --master-port ${MASTER_PORT}"
DP=$((NPROC / (TP * CP * PP))); NUM_MBS=$((GBS / (MBS * DP)))
COMM_BACKEND=kernel
if [ "$QUICK" = "1" ]; then      # a few configurations per partition, short measurements
  BO_ARGS="--n-init 3 --batches 1 --acq-batch 1 --measure-s 0.05 --cooldown-s 0 --freqs 1500 1200"
  PERSEUS_ARGS="--freqs 1500 1200 --steps 2 --skip 1"; SKIP=1; TAKE=$((STEPS - 1)); MAXIT="--max-iterations 30"
  if [ "$(python -c 'import torch; print(int(torch.cuda.is_available()))')" = "0" ]; then
    [ "$TP_COMM" = "sp_fused" ] && TP_COMM=sp          # the fused kernels need GPUs
    BO_ARGS="$BO_ARGS --comm-backend nccl"; COMM_BACKEND=nccl
  fi
else
  BO_ARGS=""; PERSEUS_ARGS=""; SKIP=10; TAKE=20; MAXIT=""
fi
mkdir -p "$WORK"

if [ "$SKIP_PROFILING" != "true" ]; then
  if [ "$TP" -gt 1 ]; then
    echo "== 1. profile every partition of the tensor-parallel path, then the non-partition pieces"
    $RUNP -m kareus_b200.cli.run_bayesian --partition all --tp-comm "$TP_COMM" -m "$MODEL" -w "$NPROF" -tp "$TP" -cp "$CP" \
        -b "$MBS" -s "$SEQ" --gpu_type "$GPU_TYPE" --clock-mode "$CLOCK_MODE" --out "$WORK/bayesian" $BO_ARGS
    $RUNP -m kareus_b200.cli.run_bayesian --nonpartition -m "$MODEL" -w "$NPROF" -tp "$TP" -cp "$CP" -b "$MBS" -s "$SEQ" \
        --gpu_type "$GPU_TYPE" --clock-mode "$CLOCK_MODE" --out "$WORK/bayesian" $BO_ARGS
  else
    echo "== 1. no tensor parallelism: the partition plan (overlap of tensor-parallel collectives) does not apply"
  fi
  echo "== 2. per-instruction time/energy at every clock for the frequency-only baselines"
  for METHOD in $PERSEUS_METHODS; do
    $RUN -m kareus_b200.cli.run_perseus_profile --method $METHOD --model "$MODEL" --tp "$TP" --pp "$PP" --mbs "$MBS" \
        --gbs "$GBS" --seq "$SEQ" --gpu_type "$GPU_TYPE" --clock-mode "$CLOCK_MODE" --out "$WORK/${METHOD}_profile.csv" \
        $PERSEUS_ARGS
  done
fi

echo "== 3. baselines: one nanobatch, two nanobatches"
for METHOD in megatron nanobatch; do
  $RUN -m kareus_b200.cli.run_train --method $METHOD --model "$MODEL" --tp "$TP" --pp "$PP" --cp "$CP" --mbs "$MBS" \
      --gbs "$GBS" --seq "$SEQ" --steps "$STEPS" --tp-comm "$TP_COMM" --clock-mode "$CLOCK_MODE" --out "$WORK/runs"
done

COMPARE="$WORK/runs/$MODEL/$TAG/nanobatch"
for METHOD in $PERSEUS_METHODS; do
  [ -f "$WORK/${METHOD}_profile.csv" ] || continue
  echo "== 4a. $METHOD: frequency-only plan from the per-instruction profile, train under its max-throughput point"
  python -m kareus_b200.cli.run_optimization --inst_profile "$WORK/${METHOD}_profile.csv" \
      --output_dir "$WORK/${METHOD}_plans" --num_stages "$PP" --num_mbs "$NUM_MBS" --gpu_type "$GPU_TYPE" \
      ${MAXIT/--max-iterations/--max_iterations}
  FREQS=$(ls "$WORK/${METHOD}_plans"/freqs_pipeline_*.py | sort | tail -1)    # the highest-numbered plan is the fastest
  $RUN -m kareus_b200.cli.run_train --method $METHOD --model "$MODEL" --tp "$TP" --pp "$PP" --cp "$CP" --mbs "$MBS" \
      --gbs "$GBS" --seq "$SEQ" --steps "$STEPS" --tp-comm "$TP_COMM" --clock-mode "$CLOCK_MODE" --freqs "$FREQS" \
      --out "$WORK/runs"
  COMPARE="$COMPARE $WORK/runs/$MODEL/$TAG/$METHOD"
  if [ "$FRONTIER" = "true" ]; then     # one more run per sampled plan: <method>/frontier/pipeline_NNNNN
    $RUN -m kareus_b200.cli.run_frontier --method $METHOD --plans-dir "$WORK/${METHOD}_plans" --model "$MODEL" --tp "$TP" \
        --pp "$PP" --cp "$CP" --mbs "$MBS" --gbs "$GBS" --seq "$SEQ" --steps "$STEPS" --tp-comm "$TP_COMM" \
        --comm-backend "$COMM_BACKEND" --clock-mode "$CLOCK_MODE" --out "$WORK/runs"
  fi
done
if [ "$TP" -gt 1 ]; then
  echo "== 4b. compose the partition frontiers, plan, train under the max-throughput plan"
  $RUN -m kareus_b200.cli.run_kareus --model "$MODEL" --tp "$TP" --pp "$PP" --cp "$CP" --mbs "$MBS" --gbs "$GBS" --seq "$SEQ" \
      --steps "$STEPS" --bayesian-dir "$WORK/bayesian" --workdir "$WORK/runs" --gpu_type "$GPU_TYPE" \
      --clock-mode "$CLOCK_MODE" --tp-comm "$TP_COMM" $MAXIT
  COMPARE="$COMPARE $WORK/runs/$MODEL/$TAG/kareus"
fi

echo "== 5. energy and time of each method against the one-nanobatch baseline"
python -m kareus_b200.cli.compare --base "$WORK/runs/$MODEL/$TAG/megatron" --runs $COMPARE --skip "$SKIP" --take "$TAKE" \
    --num_stages "$PP" --gpu_type "$GPU_TYPE"
python -m kareus_b200.cli.compare --root "$WORK/runs" --skip "$SKIP" --take "$TAKE"
if [ "$FRONTIER" = "true" ]; then
  echo "== 6. measured frontiers against the frequency-only frontier"
  python -m kareus_b200.cli.compare --root "$WORK/runs" --frontier --skip "$SKIP" --take "$TAKE"
fi
