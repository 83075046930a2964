# Build image for piper_b200: CUDA 12.9 toolchain (nvcc with sm_100a support) plus PyTorch.
FROM nvidia/cuda:12.9.1-devel-ubuntu24.04

RUN apt-get update && apt-get install -y --no-install-recommends \
      python3 python3-pip python3-venv git graphviz ninja-build && \
    rm -rf /var/lib/apt/lists/*

WORKDIR /workspace/piper_b200
COPY requirements.txt pyproject.toml ./
RUN python3 -m venv /opt/venv && /opt/venv/bin/pip install --upgrade pip && \
    /opt/venv/bin/pip install -r requirements.txt
ENV PATH=/opt/venv/bin:$PATH

COPY . .
# Compile the sm_100a kernel library in-tree (no GPU needed for the build).
RUN python -c "import __graft_entry__ as g; g.build()"

CMD ["python", "examples/test_harness.py", "--help"]
