# Image for building and running msamp on NVIDIA B200 (sm_100a).
# The reference ships NGC-based images that also build MSCCL and Transformer Engine
# (dockerfile/torch2.1-cuda12.2.dockerfile); none of that is needed here: stock NCCL and one nvcc build.
FROM nvcr.io/nvidia/pytorch:25.06-py3

ENV DEBIAN_FRONTEND=noninteractive
WORKDIR /opt/msamp
COPY . /opt/msamp

# nvcc -gencode arch=compute_100a,code=sm_100a; the shared library is built in-tree
RUN python -m pip install --no-cache-dir numpy pytest && \
    python -m msamp.ops.build && \
    python -m pip install --no-cache-dir --no-build-isolation -e .

CMD ["python", "-m", "pytest", "tests", "-q", "-m", "not gpu"]
