#!/bin/bash
# Serve a random-init Qwen3.6-35B-A3B on the visible GPU(s) and drive it with bench/serve_bench.py.
#
#   bench/run_serving_configs.sh decode      # batch 1 / 8 / 32 / 128 (BATCHES=...), 1024-token prompts, 512 output tokens
#   bench/run_serving_configs.sh sessions    # multi-round chat sessions (Poisson arrivals, growing contexts)
#   bench/run_serving_configs.sh trace       # replay of bench/sample_trace.csv with 8 session slots
#   bench/run_serving_configs.sh long        # one 131072-token prompt prefilled in 8192-token chunks (TTFT)
#
# MODEL / VOCAB name another model (random:tiny with VOCAB=1000 runs on CPU). Extra server flags go in SERVER_FLAGS (e.g. "--gpus-per-replica 2"); results are appended as JSON lines to
# ${OUT:-serve_results.jsonl}. Greedy, ignore_eos, exact output lengths; timing is taken on the client.
set -u
MODE=${1:-decode}
PORT=${PORT:-8123}
OUT=${OUT:-serve_results.jsonl}
ROOT=$(cd "$(dirname "$0")/.." && pwd)
URL=http://127.0.0.1:$PORT
case $MODE in
  long) LEN=140000; CHUNK=8192; SEQS=4 ;;
  sessions|trace) LEN=${MAX_MODEL_LEN:-40000}; CHUNK=2048; SEQS=${MAX_SEQS:-64} ;;
  *) LEN=4096; CHUNK=2048; SEQS=128 ;;
esac
# the server runs in its own process group (front, replicas, follower ranks), which is ended as a whole at exit;
# every client run and the wait for /health are bounded, so the script always ends by itself
ENGINE_MTP=${ENGINE_MTP:-0} setsid python "$ROOT/main.py" --model ${MODEL:-random:qwen36} --served-model-name q --port "$PORT" \
  --max-model-len $LEN --prefill-chunk-tokens $CHUNK --max-seqs $SEQS ${SERVER_FLAGS:-} > "${OUT%.jsonl}.server.log" 2>&1 &
SERVER=$!
trap 'kill -- -$SERVER 2>/dev/null; sleep 2; kill -9 -- -$SERVER 2>/dev/null; wait $SERVER 2>/dev/null' EXIT
UP=0
for _ in $(seq 1 ${HEALTH_WAIT:-600}); do curl -s -m 2 -o /dev/null "$URL/health" && UP=1 && break; sleep 1; done
if [ $UP = 0 ]; then echo "server did not come up" >> "$OUT"; tail -5 "${OUT%.jsonl}.server.log" >> "$OUT"; cat "$OUT"; exit 1; fi
B="timeout ${CLIENT_TIMEOUT:-900} python $ROOT/bench/serve_bench.py --url $URL --model q --vocab ${VOCAB:-248320}"
run() { echo "{\"config\": \"$1\"}" >> "$OUT"; shift; "$@" >> "$OUT" 2>&1; }
case $MODE in
  decode)
    for c in ${BATCHES:-1 8 32 128}; do
      run "decode bs$c 1024 in / 512 out" $B --concurrency $c --requests $c --prompt-len 1024 --output-len 512
    done ;;
  sessions)
    run "sessions ${SESSIONS:-16} x 4-8 rounds, first ~${FIRST:-6000} tokens, +100-2000 per round, 50-800 out, ${RATE:-4}/s" \
      $B --concurrency ${SESSIONS:-16} --sessions ${SESSIONS:-16} --rounds 4-8 --rate ${RATE:-4} --first-len ${FIRST:-6000} \
      --max-first-len $((LEN / 2)) --grow 100-2000 --output-len 50-800 ;;
  trace)
    run "trace replay, 8 slots" $B --concurrency 8 --trace "$ROOT/bench/sample_trace.csv" ;;
  long)
    run "long prefill 131072 tokens, 8192-token chunks" $B --concurrency 1 --requests 1 --prompt-len 131072 --output-len 16 ;;
esac
curl -s -m 5 "$URL/health" | cut -c1-1500 >> "$OUT"
echo >> "$OUT"
cat "$OUT"
