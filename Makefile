# In-tree build: a static archive with everything (host C++ and sm_100a kernels), the Python
# extension, the C++ test binary and the benchmark binaries. `make -j` is what
# __graft_entry__.build() runs; nvcc cross-compiles for sm_100a without a GPU present.
CUDA_HOME ?= /usr/local/cuda
PYTHON ?= python
# The system compiler links libstdc++ dynamically, like PyTorch; a toolchain that links it
# statically would put a second copy of the C++ runtime into the Python process.
CXX := $(shell command -v /usr/bin/g++ || echo g++)
NVCC ?= $(CUDA_HOME)/bin/nvcc

BUILD := build
CXXFLAGS := -std=c++17 -O2 -g -fPIC -Wall -Wno-unused-function -Wno-sign-compare -pthread \
            -Iinclude -Isrc -I$(CUDA_HOME)/include
NVCCFLAGS := -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -lineinfo \
             -Xcompiler -fPIC -Iinclude -Isrc --expt-relaxed-constexpr
LDLIBS := -L$(CUDA_HOME)/lib64 -lcudart_static -ldl -lrt -lpthread

# make SANITIZE=thread BUILD=build-tsan build-tsan/bin/tpb_test   (or SANITIZE=address): the host code
# of the library and of the C++ tests under a sanitizer, as the reference's cmake/Sanitize.cmake does.
ifdef SANITIZE
CXXFLAGS += -fsanitize=$(SANITIZE) -fno-omit-frame-pointer -O1
NVCCFLAGS += -Xcompiler -fsanitize=$(SANITIZE)
LDLIBS += -fsanitize=$(SANITIZE)
endif

# make DEBUG_KERNELS=1 BUILD=build-dbg build-dbg/bin/tpb_test: kernels that check every address they
# compute against their table entry and count what lies outside (see src/kernels/push.h).
ifdef DEBUG_KERNELS
NVCCFLAGS += -DTPB_DEBUG_KERNELS
endif

PYINC := $(shell $(PYTHON) -c "import sysconfig,pybind11;print('-I'+sysconfig.get_paths()['include'],'-I'+pybind11.get_include())")
PYEXT := $(shell $(PYTHON) -c "import sysconfig;print(sysconfig.get_config_var('EXT_SUFFIX'))")

LIB_CC := $(shell find src -name '*.cc' | sort)
LIB_CU := $(shell find src -name '*.cu' | sort)
LIB_OBJ := $(LIB_CC:%.cc=$(BUILD)/%.o) $(LIB_CU:%.cu=$(BUILD)/%.cu.o)

TEST_CC := $(shell find tests/cpp -name '*.cc' | sort)
TEST_CU := $(shell find tests/cpp -name '*.cu' | sort)
TEST_OBJ := $(TEST_CC:%.cc=$(BUILD)/%.o) $(TEST_CU:%.cu=$(BUILD)/%.cu.o)

BENCH_SRC := $(shell find benchmarks -name '*.cc' | sort)
BENCH_BIN := $(BENCH_SRC:benchmarks/%.cc=$(BUILD)/bin/%)

PYMOD := tensorpipe_b200/_C$(PYEXT)

all: $(BUILD)/libtpb.a $(PYMOD) $(BUILD)/bin/tpb_test $(BENCH_BIN)

$(BUILD)/%.o: %.cc
	@mkdir -p $(dir $@)
	$(CXX) $(CXXFLAGS) -MMD -MP -c $< -o $@

$(BUILD)/%.cu.o: %.cu
	@mkdir -p $(dir $@)
	$(NVCC) $(NVCCFLAGS) -MMD -MP -c $< -o $@

$(BUILD)/libtpb.a: $(LIB_OBJ)
	@rm -f $@
	ar rcs $@ $^

$(BUILD)/python/bindings.o: python/bindings.cc
	@mkdir -p $(dir $@)
	$(CXX) $(CXXFLAGS) $(PYINC) -fvisibility=hidden -MMD -MP -c $< -o $@

$(PYMOD): $(BUILD)/python/bindings.o $(BUILD)/libtpb.a
	$(CXX) -shared -o $@ $< -Wl,--whole-archive $(BUILD)/libtpb.a -Wl,--no-whole-archive $(LDLIBS)

$(BUILD)/bin/tpb_test: $(TEST_OBJ) $(BUILD)/libtpb.a
	@mkdir -p $(dir $@)
	$(CXX) -o $@ $(TEST_OBJ) $(BUILD)/libtpb.a $(LDLIBS)

$(BUILD)/bin/%: $(BUILD)/benchmarks/%.o $(BUILD)/libtpb.a
	@mkdir -p $(dir $@)
	$(CXX) -o $@ $< $(BUILD)/libtpb.a $(LDLIBS)

clean:
	rm -rf $(BUILD) tensorpipe_b200/_C*.so

-include $(shell find $(BUILD) -name '*.d' 2>/dev/null)

.PHONY: all clean
.SECONDARY:
