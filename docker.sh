#!/usr/bin/env bash
# Image helper for khaosz_b200 (same verbs as the reference's scripts/docker.sh:
# build | run | push | remove | info | logs).
#
#   ./docker.sh build  [-t TAG] [-f DOCKERFILE]
#   ./docker.sh run    [-t TAG] [-p PORT] [-m PARAM_DIR] [-g GPUS] [-- server flags]
#   ./docker.sh push   [-t TAG] -r REGISTRY
#   ./docker.sh remove [-t TAG]
#   ./docker.sh info   [-t TAG]
#   ./docker.sh logs   CONTAINER
set -euo pipefail

NAME=khaosz_b200
TAG=latest
DOCKERFILE=Dockerfile
PORT=8000
PARAMS="$PWD/params"
GPUS=all
REGISTRY=""

die() { echo "docker.sh: $*" >&2; exit 1; }
need_docker() { command -v docker >/dev/null 2>&1 || die "docker is not installed"; }

verb="${1:-}"; [ -n "$verb" ] || { sed -n '2,12p' "$0"; exit 1; }
shift
extra=()
while [ $# -gt 0 ]; do
    case "$1" in
        -t) TAG="$2"; shift 2 ;;
        -f) DOCKERFILE="$2"; shift 2 ;;
        -p) PORT="$2"; shift 2 ;;
        -m) PARAMS="$2"; shift 2 ;;
        -g) GPUS="$2"; shift 2 ;;
        -r) REGISTRY="$2"; shift 2 ;;
        --) shift; extra=("$@"); break ;;
        *)  extra+=("$1"); shift ;;
    esac
done
IMAGE="$NAME:$TAG"

case "$verb" in
    build)
        need_docker
        [ -f "$DOCKERFILE" ] || die "no such Dockerfile: $DOCKERFILE"
        docker build -t "$IMAGE" -f "$DOCKERFILE" .
        ;;
    run)
        need_docker
        [ -d "$PARAMS" ] || die "parameter directory not found: $PARAMS (config.json, model.safetensors, tokenizer files)"
        # one container serves on all visible GPUs when --tp_size is among the server flags
        docker run --rm -d --gpus "$GPUS" --ipc=host -p "$PORT:8000" -v "$PARAMS:/app/params:ro" "$IMAGE" \
            python -m khaosz_b200.cli.server --host 0.0.0.0 --port 8000 --device cuda --param_path /app/params "${extra[@]}"
        ;;
    push)
        need_docker
        [ -n "$REGISTRY" ] || die "push needs -r REGISTRY"
        docker tag "$IMAGE" "$REGISTRY/$IMAGE"
        docker push "$REGISTRY/$IMAGE"
        ;;
    remove)
        need_docker
        docker rmi "$IMAGE"
        ;;
    info)
        need_docker
        docker image inspect "$IMAGE" --format 'id={{.Id}} created={{.Created}} size={{.Size}}'
        ;;
    logs)
        need_docker
        [ ${#extra[@]} -ge 1 ] || die "logs needs a container id or name"
        docker logs -f "${extra[0]}"
        ;;
    *)
        die "unknown verb '$verb' (build | run | push | remove | info | logs)"
        ;;
esac
