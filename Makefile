# Top-level targets under the names the reference's makefile uses (GEMM/makefile:29-49), so that its workflow --
# `make gemm && make gemm_test`, `make gemm_run`, `./testbench.sh` (which calls ./out/gemm) -- runs here as shipped:
#
#   make lib                      the library for sm_100a (tensor-core-fp8_b200/csrc) and the CPU oracle
#   make gemm REF=<reference>     out/gemm: the reference's UNMODIFIED driver GEMM/gemm_main.cpp, compiled from where it
#                                 lies and linked against this library's gemm::GEMM / gemm::GEMM4 (replaces the
#                                 reference's own bin/gemm.o); also creates data/, which its CSV recording needs
#   make gemm_test / gemm_run     the reference's two run targets, same arguments
#   make cublas REF=<reference>   out/cublas: the reference's cuBLASLt comparator GEMM/src/cublas.cu, compiled in place
#   make cublas_run
#   make clean
#
# Nothing of the reference is copied into this repository: REF names its checkout.
NVCC     ?= /usr/local/cuda/bin/nvcc
CUDA     ?= /usr/local/cuda
HOSTCXX  ?= g++
REF      ?=
ROOT     := $(dir $(abspath $(lastword $(MAKEFILE_LIST))))
LIBDIR   := $(ROOT)tensor-core-fp8_b200/csrc
OUT_DIR  := $(ROOT)out
OBJ_DIR  := $(ROOT)bin
RECORD_DIR := $(ROOT)data

.PHONY: lib gemm gemm_test gemm_run cublas cublas_run clean need_ref
lib:
	$(MAKE) -s -C $(LIBDIR) all
	$(MAKE) -s -C $(ROOT)oracle oracle

need_ref:
	@if [ -z "$(REF)" ] || [ ! -f "$(REF)/GEMM/gemm_main.cpp" ]; then echo "REF=<root of the reference checkout> is required"; exit 2; fi

$(OUT_DIR) $(OBJ_DIR) $(RECORD_DIR):
	mkdir -p $@

gemm: need_ref lib | $(OUT_DIR) $(OBJ_DIR) $(RECORD_DIR)
	$(HOSTCXX) -O2 -std=c++17 -w -I$(CUDA)/include -c $(REF)/GEMM/gemm_main.cpp -o $(OBJ_DIR)/gemm_main.o
	$(HOSTCXX) -o $(OUT_DIR)/gemm $(OBJ_DIR)/gemm_main.o -L$(LIBDIR) -lb200fp8 -L$(CUDA)/lib64 -lcudart \
	    -Wl,-rpath,$(LIBDIR) -Wl,-rpath,$(CUDA)/lib64

gemm_test:
	cd $(ROOT) && $(OUT_DIR)/gemm 128 128 128 2 1 0 0
gemm_run:
	cd $(ROOT) && $(OUT_DIR)/gemm 4096 4096 4096 1 0 0 0

cublas: need_ref | $(OUT_DIR)
	$(NVCC) -w -gencode arch=compute_100a,code=sm_100a -lcublasLt $(REF)/GEMM/src/cublas.cu -o $(OUT_DIR)/cublas
cublas_run:
	$(OUT_DIR)/cublas 100

clean:
	rm -rf $(OBJ_DIR) $(OUT_DIR) $(RECORD_DIR)
	$(MAKE) -s -C $(LIBDIR) clean
