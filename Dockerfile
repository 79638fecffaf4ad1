# Build and run image for B200 (sm_100a).  nvcc in the base image compiles the kernels at build time; no GPU is
# needed to build.
FROM nvcr.io/nvidia/pytorch:25.09-py3
WORKDIR /opt/areno_b200
COPY pyproject.toml README.md ./
COPY areno_b200 ./areno_b200
COPY examples ./examples
COPY bench.py __graft_entry__.py ./
RUN python -m pip install --no-cache-dir -e ".[serve,data,metrics]" \
 && python -m areno_b200.build
ENV NCCL_NVLS_ENABLE=1
ENTRYPOINT ["areno"]
CMD ["check"]
