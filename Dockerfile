# distca_b200 in a container: any CUDA >= 12.8 PyTorch image whose nvcc knows sm_100a will do.
# (the reference builds on nvcr.io/nvidia/pytorch:24.12-py3 and then installs Megatron-LM, TransformerEngine,
#  flash-attn and NVSHMEM on top, Dockerfile + scripts/docker_install_and_build.sh; none of them is needed here)
ARG BASE=nvcr.io/nvidia/pytorch:25.04-py3
FROM ${BASE}
WORKDIR /workspace/distca_b200
COPY . .
# builds _kernels.so (nvcc -gencode arch=compute_100a,code=sm_100a) and the C++ planner, then installs the package
RUN python -m pip install --no-build-isolation --no-deps -e . \
 && python -c "import __graft_entry__ as g; g.build()"
# CPU part of the test-suite as the image's self-check (no GPU at build time)
RUN python -m pytest tests -q -x -m "not gpu" -k "planner or tools or source_rules"
ENV NCCL_NVLS_ENABLE=0
CMD ["bash", "examples/single_gpu_smoke.sh"]
