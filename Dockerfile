# Image for serving on B200 (sm_100a).  Build stage: CUDA 12.9 toolchain, the Python environment and the in-tree
# compile of the kernel library (nvcc cross-compiles for sm_100a, so the build needs no GPU).  Runtime stage: the same
# CUDA base with the prepared environment; `python -m minisgl` is the entry point (OpenAI-compatible server).
ARG CUDA_VERSION=12.9.1
ARG UBUNTU_VERSION=24.04
ARG PYTHON_VERSION=3.12

FROM nvidia/cuda:${CUDA_VERSION}-devel-ubuntu${UBUNTU_VERSION} AS builder
ARG PYTHON_VERSION
RUN apt-get update && apt-get install -y --no-install-recommends \
        python${PYTHON_VERSION} python${PYTHON_VERSION}-dev python${PYTHON_VERSION}-venv python3-pip g++ \
    && rm -rf /var/lib/apt/lists/*
WORKDIR /app
COPY setup.py pyproject.toml README.md ./
COPY deepseek-v4-sm80_b200/ ./deepseek-v4-sm80_b200/
COPY minisgl/ ./minisgl/
RUN python${PYTHON_VERSION} -m venv /app/.venv \
    && . /app/.venv/bin/activate \
    && pip install --no-cache-dir torch numpy safetensors transformers fastapi uvicorn pyzmq msgpack httpx \
    && python deepseek-v4-sm80_b200/ops/build.py \
    && pip install --no-cache-dir --no-build-isolation -e .

FROM nvidia/cuda:${CUDA_VERSION}-devel-ubuntu${UBUNTU_VERSION} AS runtime
ARG PYTHON_VERSION
RUN apt-get update && apt-get install -y --no-install-recommends \
        python${PYTHON_VERSION} python${PYTHON_VERSION}-venv \
    && rm -rf /var/lib/apt/lists/*
WORKDIR /app
COPY --from=builder /app /app
ENV PATH="/app/.venv/bin:${PATH}" \
    NCCL_DEBUG=WARN
EXPOSE 1919
ENTRYPOINT ["python", "-m", "minisgl"]
CMD ["--help"]
