# Native artefacts without Python: the ncclNet plugin, the monitor daemon, the two-process harness and the C library
# with the sm_100a kernels.  Target names follow the reference's Makefile (`make fl`, `make monitor`, Makefile:33-49);
# `python -m fuselink_b200.build` builds the same files (plus the torch extension) and is what the tests use.
#
#   make fl        build/lib/libnccl-net-fuselink.so      NCCL_NET_PLUGIN=fuselink, LD_LIBRARY_PATH=$PWD/build/lib
#   make monitor   build/bin/fuselink-monitor
#   make harness   build/bin/fl_net_harness
#   make lib       build/lib/libfuselink.so               kernels + cuMem regions + monitor (include/fuselink.h); needs nvcc
#   make all       everything above;  make clean;  make test (CPU tier of the tests; needs Python)
CXX      ?= g++
NVCC     ?= /usr/local/cuda/bin/nvcc
CUDA_HOME ?= /usr/local/cuda
OPT      ?= -O2 -g
CXXFLAGS := $(OPT) -std=c++17 -fPIC -Wall -Wno-unused-function -pthread -I$(CUDA_HOME)/include
NVCCFLAGS ?= -gencode arch=compute_100a,code=sm_100a -lineinfo -O3 -std=c++17 -Xcompiler -fPIC --expt-relaxed-constexpr

SRC   := fuselink_b200/csrc
BUILD := build
OBJ   := $(BUILD)/obj

NET_SRCS  := $(wildcard $(SRC)/net/*.cc)
NET_SRCS  := $(filter-out $(SRC)/net/harness_main.cc,$(NET_SRCS))
NET_OBJS  := $(patsubst $(SRC)/net/%.cc,$(OBJ)/net_%.o,$(NET_SRCS))
HOST_OBJS := $(OBJ)/vmm.o $(OBJ)/monitor.o
CU_SRCS   := $(wildcard $(SRC)/kernels/*.cu)
CU_OBJS   := $(patsubst $(SRC)/kernels/%.cu,$(OBJ)/%.o,$(CU_SRCS))
HEADERS   := $(wildcard $(SRC)/*/*.h) $(wildcard $(SRC)/*/*.cuh)

.PHONY: all fl monitor harness lib clean test
all: fl monitor harness lib
fl: $(BUILD)/lib/libnccl-net-fuselink.so
monitor: $(BUILD)/bin/fuselink-monitor
harness: $(BUILD)/bin/fl_net_harness
lib: $(BUILD)/lib/libfuselink.so

$(OBJ) $(BUILD)/lib $(BUILD)/bin:
	mkdir -p $@

$(OBJ)/net_%.o: $(SRC)/net/%.cc $(HEADERS) | $(OBJ)
	$(CXX) $(CXXFLAGS) -c $< -o $@
$(OBJ)/vmm.o: $(SRC)/mem/vmm.cc $(HEADERS) | $(OBJ)
	$(CXX) $(CXXFLAGS) -c $< -o $@
$(OBJ)/monitor.o: $(SRC)/monitor/monitor.cc $(HEADERS) | $(OBJ)
	$(CXX) $(CXXFLAGS) -c $< -o $@
$(OBJ)/%.o: $(SRC)/kernels/%.cu $(HEADERS) | $(OBJ)
	$(NVCC) $(NVCCFLAGS) -c $< -o $@

# libcuda and libibverbs are opened at run time (dlopen): the plugin links neither, unlike the reference's
# `-libverbs -lnccl -lcuda` (Makefile:14)
$(BUILD)/lib/libnccl-net-fuselink.so: $(NET_OBJS) $(HOST_OBJS) | $(BUILD)/lib
	$(CXX) -shared -Wl,-soname,libnccl-net-fuselink.so -o $@ $^ -ldl -lrt -lpthread
$(BUILD)/bin/fuselink-monitor: $(SRC)/monitor/monitor_main.cc $(OBJ)/monitor.o | $(BUILD)/bin
	$(CXX) $(CXXFLAGS) -o $@ $^ -lrt -lpthread
$(BUILD)/bin/fl_net_harness: $(SRC)/net/harness_main.cc | $(BUILD)/bin
	$(CXX) $(CXXFLAGS) -o $@ $< -ldl -lpthread
$(BUILD)/lib/libfuselink.so: $(CU_OBJS) $(HOST_OBJS) | $(BUILD)/lib
	$(CXX) -shared -o $@ $^ -L$(CUDA_HOME)/lib64 -Wl,-rpath,$(CUDA_HOME)/lib64 -lcudart -ldl -lrt -lpthread

# the CPU tier of the tests (the reference declares a `test` target and gives it no rule, Makefile:16)
test:
	python -m fuselink_b200.build
	python -m pytest tests -q -m "not gpu"

clean:
	rm -rf $(BUILD)
