# Configuration fragment for projects that build against this library with make: include it
# after setting PS_PATH (the root of this repository) and, optionally, USE_KEY32.
#
#   PS_PATH := third_party/ps_lite_b200
#   include $(PS_PATH)/make/ps.mk
#   myprog: myprog.cc $(PS_LIB_A)
#   	$(CXX) $(CXXFLAGS) $(PS_CFLAGS) $< $(PS_LDFLAGS_A) -o $@
#
# The variable names PS_LDFLAGS_SO / PS_LDFLAGS_A and the ADD_CFLAGS convention are those of the
# reference's make/ps.mk; there they name protobuf and ZeroMQ, which this runtime does not need.
ADD_CFLAGS += $(if $(filter 1,$(USE_KEY32)),-DUSE_KEY32=1)

PS_PATH ?= .
PS_CFLAGS = -std=c++17 -pthread -I$(PS_PATH)/include $(ADD_CFLAGS)
PS_LIB_A = $(PS_PATH)/build/make/libps.a
PS_LIB_SO = $(PS_PATH)/build/make/libpsb200_core.so
PS_LDFLAGS_A = $(PS_LIB_A) -pthread -ldl
PS_LDFLAGS_SO = -L$(PS_PATH)/build/make -lpsb200_core -Wl,-rpath,$(abspath $(PS_PATH)/build/make) -pthread -ldl
