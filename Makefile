# Build contract of the reference (its Makefile:11-21), kept so that existing
# wrappers that run `make -s lib` and load build/libtinytorch.so keep working:
#   make lib     -> build/libtinytorch.so   (also tinytorch_b200/libtinytorch.so)
#   make pybind  -> build/tinytorch_pybind<ext-suffix>
# Everything is compiled for sm_100a only; there is no CPU path.
NVCC    ?= /usr/local/cuda/bin/nvcc
HOSTCXX ?= /usr/bin/g++
ARCH    := -gencode arch=compute_100a,code=sm_100a
# EXTRA=-DTT_TUNING builds the library with its timing aids and TT_TC_* environment knobs (never for production)
EXTRA   ?=
NVFLAGS := $(ARCH) -O3 -std=c++17 -lineinfo -Xcompiler -fPIC -ccbin $(HOSTCXX) -Iinclude -Itinytorch_b200/csrc $(EXTRA)
SRC     := tinytorch_b200/csrc
BUILD   := build
OBJDIR  := $(BUILD)/obj
# -fmad=false: the exact-fp32 and elementwise kernels round every multiply and
# add separately, like the reference's C; only explicit fmaf() fuses.
EXACT   := context tensor ops autograd dist peer_reduce kernels_elementwise kernels_spatial kernels_pipeline gemm_simt
FAST    := gemm_tc conv_tc
OBJS    := $(addprefix $(OBJDIR)/,$(addsuffix .o,$(EXACT) $(FAST)))
HDRS    := $(wildcard include/*.h) $(SRC)/tt_internal.h $(SRC)/tcgen05_utils.cuh

PYBIND_INC := $(shell python3 -m pybind11 --includes 2>/dev/null)
EXT_SUFFIX := $(shell python3-config --extension-suffix 2>/dev/null || echo ".so")

lib: $(BUILD)/libtinytorch.so
pybind: $(BUILD)/tinytorch_pybind$(EXT_SUFFIX)

$(OBJDIR):
	mkdir -p $(OBJDIR)

$(addprefix $(OBJDIR)/,$(addsuffix .o,$(EXACT))): $(OBJDIR)/%.o: $(SRC)/%.cu $(HDRS) | $(OBJDIR)
	$(NVCC) $(NVFLAGS) -fmad=false -c $< -o $@

$(addprefix $(OBJDIR)/,$(addsuffix .o,$(FAST))): $(OBJDIR)/%.o: $(SRC)/%.cu $(HDRS) | $(OBJDIR)
	$(NVCC) $(NVFLAGS) -c $< -o $@

tinytorch_b200/libtinytorch.so: $(OBJS)
	$(NVCC) $(ARCH) -shared -ccbin $(HOSTCXX) -o $@ $(OBJS) -cudart static -ldl -lrt -lpthread

$(BUILD)/libtinytorch.so: tinytorch_b200/libtinytorch.so
	cp -f $< $@

$(BUILD)/tinytorch_pybind$(EXT_SUFFIX): $(SRC)/bindings.cpp $(BUILD)/libtinytorch.so $(HDRS)
	$(HOSTCXX) -O2 -std=c++17 -fPIC -shared $(PYBIND_INC) -Iinclude -o $@ $(SRC)/bindings.cpp \
	    -L$(BUILD) -ltinytorch -Wl,-rpath,'$$ORIGIN'

clean:
	rm -rf $(BUILD) tinytorch_b200/libtinytorch.so

.PHONY: lib pybind clean
