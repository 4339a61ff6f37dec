# khaosz_b200: CUDA 12.9 devel image (nvcc is needed to build the sm_100a kernel library in-tree)
FROM nvidia/cuda:12.9.1-devel-ubuntu24.04

ENV DEBIAN_FRONTEND=noninteractive PIP_NO_CACHE_DIR=1
RUN apt-get update && apt-get install -y --no-install-recommends python3.12 python3.12-venv python3-pip curl \
    && rm -rf /var/lib/apt/lists/*
RUN python3.12 -m venv /opt/venv
ENV PATH="/opt/venv/bin:$PATH"

WORKDIR /app
RUN pip install torch --index-url https://download.pytorch.org/whl/cu128 \
    && pip install safetensors tokenizers jinja2 fastapi uvicorn pydantic numpy tqdm
COPY khaosz_b200/ ./khaosz_b200/
COPY __graft_entry__.py bench.py ./
# compile every kernel for sm_100a (cross-compiles without a GPU)
RUN python -c "import __graft_entry__ as g; g.build()"

EXPOSE 8000
HEALTHCHECK --interval=30s --timeout=10s --start-period=60s --retries=3 CMD curl -f http://localhost:8000/health || exit 1
CMD ["python", "-m", "khaosz_b200.cli.server", "--port", "8000", "--device", "cuda", "--param_path", "/app/params"]
