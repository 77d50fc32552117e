# Image for 8 x B200 nodes: CUDA 12.9 toolchain (nvcc with sm_100a), PyTorch with NCCL, this package built in-tree.
FROM nvidia/cuda:12.9.0-devel-ubuntu24.04

ENV DEBIAN_FRONTEND=noninteractive
RUN apt-get update && apt-get install -y --no-install-recommends \
        python3 python3-pip python3-venv git pdsh openssh-client && \
    rm -rf /var/lib/apt/lists/*

RUN python3 -m venv /opt/venv
ENV PATH=/opt/venv/bin:$PATH
RUN pip install --no-cache-dir torch numpy sympy pyyaml pytest

WORKDIR /workspace
COPY . /workspace
# compiles mist_b200/csrc/*.cu for sm_100a and the C++ runtime into mist_b200/_native (needs no GPU)
RUN pip install --no-cache-dir -e .

# quick check that does not need a GPU
RUN python benchmark/mist_b200/analysis/run.py experiment=b200-gpt3-2.7b-dp8-zero2 output_dir=/tmp/analysis
