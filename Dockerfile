# Image of the serving engine for NVIDIA B200 (sm_100a) nodes: CUDA 12.9 toolkit (nvcc is needed once, to build the
# kernel library in-tree), Python 3.12, the pinned wheels of requirements.txt, then the ahead-of-time kernel build.
# Model weights are never baked in: mount the Hugging Face cache read-only and point --model at it.
#
#   docker build -t b200serve .
#   docker run --gpus all --ipc=host -v $HF_HOME:/hf:ro -e HF_HOME=/hf -e HF_HUB_OFFLINE=1 -p 8000:8000 b200serve \
#       python main.py --model Qwen/Qwen3.6-35B-A3B --host 0.0.0.0 --port 8000
#
# --ipc=host (or a large --shm-size) is needed by the multi-GPU modes: ranks map each other's buffers through CUDA IPC.
FROM nvidia/cuda:12.9.1-devel-ubuntu24.04

RUN apt-get update \
 && apt-get install -y --no-install-recommends python3.12 python3-pip python-is-python3 \
 && rm -rf /var/lib/apt/lists/*

ENV PIP_BREAK_SYSTEM_PACKAGES=1 PIP_ROOT_USER_ACTION=ignore PYTHONUNBUFFERED=1
COPY requirements.txt /tmp/requirements.txt
RUN pip install --no-cache-dir -r /tmp/requirements.txt --extra-index-url https://download.pytorch.org/whl/cu128 \
 && rm /tmp/requirements.txt

WORKDIR /opt/b200serve
COPY . /opt/b200serve
# nvcc cross-compiles for sm_100a without a GPU: the library is part of the image, nothing is compiled while serving
RUN python -c "import __graft_entry__ as g; g.build()"

# expert-parallel and tensor-parallel replicas rendezvous on the loopback interface
ENV MASTER_ADDR=127.0.0.1 NCCL_NVLS_ENABLE=0
EXPOSE 8000
CMD ["python", "main.py", "--host", "0.0.0.0", "--port", "8000"]
