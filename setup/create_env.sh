#!/bin/bash
# Prepare an environment for lingua_b200 on a machine with CUDA >= 12.8 and a Blackwell GPU.
# (The reference's setup/create_env.sh builds a conda env and pip-installs torch, xformers and friends;
# this library needs PyTorch, numpy, pyyaml and - optionally - sentencepiece / tiktoken / pyarrow / pandas,
# and builds its own kernels.)
set -e
python -m pip install -r requirements.txt || echo "optional packages missing (no package index?): continuing"
python -c "import torch, yaml, numpy; print('torch', torch.__version__)"
python -m lingua_b200.build            # nvcc -> lingua_b200/lib/liblingua_b200.so (sm_100a)
g++ -O2 -std=c++17 -o setup/lineshuf setup/lineshuf.cpp
python -m pytest tests -q -m "not gpu" -x
