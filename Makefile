# Builds the host runtime (libps.a / libpsb200_core.so), the CUDA data plane
# (libpsb200_device.so, sm_100a) and the C++ test programs.  Python users do not need this:
# ps_lite_b200/_build.py performs the same compilations on import.
CXX ?= g++
NVCC ?= nvcc
CXXFLAGS ?= -std=c++17 -O2 -g -fPIC -Wall -pthread -Iinclude -Isrc
NVFLAGS ?= -gencode arch=compute_100a,code=sm_100a -lineinfo -O3 -std=c++17 -Xcompiler -fPIC -Iinclude -Isrc
ifdef ASAN
CXXFLAGS += -fsanitize=address -fno-omit-frame-pointer
endif
ifdef TSAN
CXXFLAGS += -fsanitize=thread
endif
ifdef USE_KEY32
CXXFLAGS += -DUSE_KEY32=1
endif

CORE_SRC := $(wildcard src/core/*.cc src/van/*.cc src/capi/*.cc)
CORE_OBJ := $(patsubst %.cc,build/make/%.o,$(CORE_SRC))
DEV_SRC := $(wildcard src/kernels/*.cu src/device/*.cu)
DEV_OBJ := $(patsubst %.cu,build/make/%.o,$(DEV_SRC))
TESTS := $(patsubst tests/cpp/%.cc,build/make/tests/%,$(wildcard tests/cpp/*.cc))

all: build/make/libps.a build/make/libpsb200_core.so
device: build/make/libpsb200_device.so
test: $(TESTS)
	build/make/tests/unit_core
	build/make/tests/loop_kv
	build/make/tests/shm_frames
	python -m ps_lite_b200.launch.local -n 2 -s 2 build/make/tests/kv_config1

# -MMD -MP: every object records the headers it was compiled against, so that a changed header
# rebuilds what includes it
build/make/%.o: %.cc
	@mkdir -p $(dir $@)
	$(CXX) $(CXXFLAGS) -MMD -MP -c $< -o $@
build/make/%.o: %.cu
	@mkdir -p $(dir $@)
	$(NVCC) $(NVFLAGS) -c $< -o $@
build/make/libps.a: $(CORE_OBJ)
	ar crv $@ $^ > /dev/null
build/make/libpsb200_core.so: $(CORE_OBJ)
	$(CXX) -shared -pthread -o $@ $^
build/make/libpsb200_device.so: $(DEV_OBJ)
	$(NVCC) -shared -gencode arch=compute_100a,code=sm_100a -o $@ $^ -lcudart
build/make/tests/%: tests/cpp/%.cc build/make/libps.a
	@mkdir -p $(dir $@)
	$(CXX) $(CXXFLAGS) -MMD -MP -MF $@.d $< build/make/libps.a -o $@
-include $(CORE_OBJ:.o=.d) $(addsuffix .d,$(TESTS))
lint:
	python tests/lint.py
clean:
	rm -rf build/make
.PHONY: all device test lint clean
