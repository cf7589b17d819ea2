# Image for the B200 (sm_100a) framework: CUDA 12.9 toolkit for nvcc, PyTorch with CUDA, the in-tree extension built at
# image-build time. Role of the reference's parameter-golf-rs/deploy/Dockerfile (pinned CUDA / NCCL / cuDNN, binaries built in
# a builder stage); no cuDNN or cudnn-frontend is needed here because attention and the GEMMs are this package's own kernels.
#
#   docker build -t pgb200 .
#   docker run --gpus all --ipc=host --shm-size=16g pgb200 python -m parameter_golf_b200.doctor --require-gpu
#   docker run --gpus all --ipc=host --shm-size=16g pgb200 \
#       python -m parameter_golf_b200.launch run --gpus 8 --result-json /out/run.json -- --spec specs/record_profile.toml --mode record
#
# --ipc=host: the ranks exchange CUDA IPC handles of their symmetric buffers and the data loader uses pinned host rings.
FROM nvidia/cuda:12.9.1-devel-ubuntu24.04

RUN apt-get update && apt-get install -y --no-install-recommends python3 python3-pip python3-venv ninja-build libzstd1 git && \
    rm -rf /var/lib/apt/lists/*
RUN python3 -m venv /opt/venv
ENV PATH="/opt/venv/bin:${PATH}"
RUN pip install --no-cache-dir torch numpy sentencepiece pytest

WORKDIR /workspace/parameter_golf_b200
COPY pyproject.toml setup.py README.md __graft_entry__.py bench.py ./
COPY parameter_golf_b200/ parameter_golf_b200/
COPY specs/ specs/
COPY bench/ bench/
COPY tests/ tests/

# nvcc cross-compiles for sm_100a without a GPU present
RUN python -c "import __graft_entry__ as g; g.build()"
ENV PYTHONPATH=/workspace/parameter_golf_b200
CMD ["python", "-m", "parameter_golf_b200.doctor"]
