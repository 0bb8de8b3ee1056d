# Image for training and serving on B200 machines.  The base image must provide CUDA >= 12.8 (nvcc with sm_100a).
FROM nvidia/cuda:12.9.0-devel-ubuntu24.04

RUN apt-get update && apt-get install -y --no-install-recommends python3 python3-pip python3-venv git \
    && rm -rf /var/lib/apt/lists/*
RUN python3 -m venv /opt/venv
ENV PATH=/opt/venv/bin:$PATH
RUN pip install --no-cache-dir torch --index-url https://download.pytorch.org/whl/cu128

WORKDIR /opt/dice_embeddings_b200
COPY . .
RUN pip install --no-cache-dir -r requirements.txt && pip install --no-cache-dir -e .
# compiles csrc/*.cu for sm_100a into dice_embeddings_b200/ops/libdice_b200.so (no GPU needed at build time)
RUN python -c "import __graft_entry__ as g; g.build()"

ENTRYPOINT ["dicee"]
CMD ["--help"]
