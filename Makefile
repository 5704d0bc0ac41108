# Builds the native parts: sm_100a kernels, the daemon (libmccs_daemon.so + mccsd),
# the client shim (libmccs.so), the LD_PRELOAD allocator hook, the apps and the
# host-side unit tests. Everything lands in mccs_b200/_native/.
NVCC      ?= nvcc
CXX       ?= g++
OUT       := mccs_b200/_native
OBJ       := build/obj
ARCH      := -gencode arch=compute_100a,code=sm_100a
CXXFLAGS  := -std=c++17 -O2 -g -fPIC -Wall -Wextra -Wno-unused-parameter -pthread -I/usr/local/cuda/include
NVCCFLAGS := -std=c++17 -O3 -lineinfo $(ARCH) -Xcompiler -fPIC,-Wall,-Wno-unused-parameter -Xptxas -v
LDLIBS    := -lpthread -ldl -lrt

TYPES := i8:int8_t u8:uint8_t i32:int32_t u32:uint32_t i64:int64_t u64:uint64_t f16:__half f32:float f64:double bf16:__nv_bfloat16
NVLS_TYPES := f16 f32 bf16
TYPE_OBJS := $(foreach t,$(TYPES),$(OBJ)/inst_$(word 1,$(subst :, ,$(t))).o) $(foreach t,$(TYPES),$(OBJ)/batch_$(word 1,$(subst :, ,$(t))).o)

HOST_SRCS := csrc/common/value.cc csrc/common/log.cc csrc/ipc/uds.cc csrc/device/host_backend.cc \
             csrc/daemon/config.cc csrc/daemon/transport.cc csrc/daemon/planner.cc csrc/daemon/qos.cc csrc/daemon/trace.cc \
             csrc/daemon/runtime.cc csrc/daemon/daemon.cc csrc/daemon/proxy.cc csrc/daemon/admin.cc
HOST_OBJS := $(patsubst csrc/%.cc,$(OBJ)/%.o,$(HOST_SRCS))
# the kernels compiled for the host against the SIMT emulator (used by the host backend on request)
EMU_OBJ   := $(OBJ)/device/emulated_kernels.o
CUDA_OBJS := $(OBJ)/device/cuda_backend.o $(OBJ)/kernels/launch.o $(OBJ)/kernels/untyped.o $(OBJ)/kernels/noalloc.o $(TYPE_OBJS)
SHIM_SRCS := csrc/shim/libmccs.cc csrc/common/value.cc csrc/common/log.cc csrc/ipc/uds.cc
SHIM_OBJS := $(patsubst csrc/%.cc,$(OBJ)/%.o,$(SHIM_SRCS))
HDRS := $(wildcard csrc/*/*.h csrc/*/*.cuh)

APPS := allreduce_bench allgather_bench allreduce_proto allgather_proto reducescatter_proto traffic_gen ring_config mccs_hello
APP_BINS := $(addprefix $(OUT)/,$(APPS))

all: $(OUT)/libmccs_daemon.so $(OUT)/libmccs.so $(OUT)/libmccs_kernels.so $(OUT)/mccsd $(OUT)/libmccs_preload.so $(APP_BINS) $(OUT)/host_tests

$(OBJ)/%.o: csrc/%.cc $(HDRS)
	@mkdir -p $(dir $@)
	$(CXX) $(CXXFLAGS) -c $< -o $@

$(EMU_OBJ): csrc/device/emulated_kernels.cc $(wildcard csrc/tests/sim/*.h) $(HDRS)
	@mkdir -p $(dir $@)
	$(CXX) $(CXXFLAGS) -O1 -g0 -Wno-unknown-pragmas -Wno-sign-compare -Wno-maybe-uninitialized -c $< -o $@

$(OBJ)/device/cuda_backend.o: csrc/device/cuda_backend.cu $(HDRS)
	@mkdir -p $(dir $@)
	$(NVCC) $(NVCCFLAGS) -c $< -o $@ 2> $@.log || (cat $@.log; false)

$(OBJ)/kernels/%.o: csrc/kernels/%.cu $(HDRS)
	@mkdir -p $(dir $@)
	$(NVCC) $(NVCCFLAGS) -c $< -o $@ 2> $@.log || (cat $@.log; false)

define TYPE_RULE
$(OBJ)/inst_$(1).o: csrc/kernels/inst_dtype.cu $(HDRS)
	@mkdir -p $$(dir $$@)
	$(NVCC) $(NVCCFLAGS) -DMCCS_T=$(2) -DMCCS_TNAME=$(1) $(if $(filter $(1),$(NVLS_TYPES)),-DMCCS_NVLS=1) -c $$< -o $$@ 2> $$@.log || (cat $$@.log; false)
$(OBJ)/batch_$(1).o: csrc/kernels/inst_batch.cu $(HDRS)
	@mkdir -p $$(dir $$@)
	$(NVCC) $(NVCCFLAGS) -DMCCS_T=$(2) -DMCCS_TNAME=$(1) $(if $(filter $(1),$(NVLS_TYPES)),-DMCCS_NVLS=1) -c $$< -o $$@ 2> $$@.log || (cat $$@.log; false)
endef
$(foreach t,$(TYPES),$(eval $(call TYPE_RULE,$(word 1,$(subst :, ,$(t))),$(word 2,$(subst :, ,$(t))))))

$(OUT)/libmccs_daemon.so: $(HOST_OBJS) $(EMU_OBJ) $(CUDA_OBJS) csrc/exports.map
	@mkdir -p $(OUT)
	$(NVCC) $(ARCH) -shared -cudart static -Xlinker --version-script=csrc/exports.map -o $@ $(HOST_OBJS) $(EMU_OBJ) $(CUDA_OBJS) $(LDLIBS)

# The kernels alone, for clients that launch them themselves ([b200] launch = "client").
KLIB_OBJS := $(OBJ)/kernels/client_entry.o $(OBJ)/kernels/launch.o $(OBJ)/kernels/untyped.o $(TYPE_OBJS)
$(OUT)/libmccs_kernels.so: $(KLIB_OBJS) csrc/exports_kernels.map
	@mkdir -p $(OUT)
	$(NVCC) $(ARCH) -shared -cudart static -Xlinker --version-script=csrc/exports_kernels.map -o $@ $(KLIB_OBJS) $(LDLIBS)

$(OUT)/libmccs.so: $(SHIM_OBJS) $(EMU_OBJ) csrc/exports.map
	@mkdir -p $(OUT)
	$(CXX) -shared -Wl,--version-script=csrc/exports.map -o $@ $(SHIM_OBJS) $(EMU_OBJ) $(LDLIBS)

$(OUT)/libmccs_preload.so: $(OBJ)/shim/preload.o $(OUT)/libmccs.so
	$(CXX) -shared -Wl,--version-script=csrc/exports_preload.map -o $@ $(OBJ)/shim/preload.o -L$(OUT) -lmccs -Wl,-rpath,'$$ORIGIN' $(LDLIBS)

$(OUT)/mccsd: $(OBJ)/daemon/main.o $(OUT)/libmccs_daemon.so
	$(CXX) -o $@ $(OBJ)/daemon/main.o -L$(OUT) -lmccs_daemon -Wl,-rpath,'$$ORIGIN' $(LDLIBS)

$(OUT)/%: $(OBJ)/apps/%.o $(OBJ)/apps/app_common.o $(OUT)/libmccs.so
	$(CXX) -o $@ $(OBJ)/apps/$*.o $(OBJ)/apps/app_common.o -L$(OUT) -lmccs -Wl,-rpath,'$$ORIGIN' $(LDLIBS)

$(OUT)/host_tests: $(OBJ)/tests/host_tests.o $(OUT)/libmccs_daemon.so
	$(CXX) -o $@ $(OBJ)/tests/host_tests.o -L$(OUT) -lmccs_daemon -Wl,-rpath,'$$ORIGIN' $(LDLIBS)

# Host-only builds of daemon + client library + a multi-tenant stress run in one process,
# under ThreadSanitizer / AddressSanitizer+UBSan (no GPU, no CUDA toolkit needed at run time).
SAN_SRCS := $(sort $(HOST_SRCS) $(SHIM_SRCS)) csrc/tests/no_cuda_backend.cc csrc/tests/stress_host.cc
SAN_CXX ?= /usr/bin/g++
SAN_FLAGS := -std=c++17 -O1 -g -fno-omit-frame-pointer -Wall -Wextra -Wno-unused-parameter -pthread -I/usr/local/cuda/include

build/san/stress_tsan: $(SAN_SRCS) $(HDRS)
	@mkdir -p build/san
	$(SAN_CXX) $(SAN_FLAGS) -fsanitize=thread -o $@ $(SAN_SRCS) $(LDLIBS)

build/san/stress_asan: $(SAN_SRCS) $(HDRS)
	@mkdir -p build/san
	$(SAN_CXX) $(SAN_FLAGS) -fsanitize=address,undefined -fno-sanitize-recover=undefined -o $@ $(SAN_SRCS) $(LDLIBS)

# The stand-alone daemon (host backend only) under a sanitizer, for the failure-path tests:
#   make build/san/mccsd_asan && MCCSD=build/san/mccsd_asan python -m pytest tests/test_service_features.py
SAN_DAEMON_SRCS := $(HOST_SRCS) csrc/tests/no_cuda_backend.cc csrc/daemon/main.cc
build/san/mccsd_asan: $(SAN_DAEMON_SRCS) $(HDRS)
	@mkdir -p build/san
	$(SAN_CXX) $(SAN_FLAGS) -fsanitize=address,undefined -fno-sanitize-recover=undefined -o $@ $(SAN_DAEMON_SRCS) $(LDLIBS)
build/san/mccsd_tsan: $(SAN_DAEMON_SRCS) $(HDRS)
	@mkdir -p build/san
	$(SAN_CXX) $(SAN_FLAGS) -fsanitize=thread -o $@ $(SAN_DAEMON_SRCS) $(LDLIBS)

# The collective kernels themselves on the CPU: the same .cuh sources, compiled by the host
# compiler against a SIMT emulator (csrc/tests/sim), every variant checked against plain sums.
build/sim/kernel_sim_test: csrc/tests/kernel_sim_test.cc $(wildcard csrc/tests/sim/*.h) $(HDRS)
	@mkdir -p build/sim
	$(SAN_CXX) -std=c++17 -O1 -g -Wall -Wno-unknown-pragmas -Wno-unused-parameter -pthread -I/usr/local/cuda/include -o $@ csrc/tests/kernel_sim_test.cc

simtest: build/sim/kernel_sim_test
	build/sim/kernel_sim_test

tsan: build/san/stress_tsan
	TSAN_OPTIONS="halt_on_error=0 second_deadlock_stack=1 suppressions=csrc/tests/tsan.supp" build/san/stress_tsan 40
	TSAN_OPTIONS="halt_on_error=0 second_deadlock_stack=1 suppressions=csrc/tests/tsan.supp" build/san/stress_tsan 40 memops

build/san/fuzz_value: csrc/tests/fuzz_value.cc csrc/common/value.cc csrc/common/log.cc csrc/daemon/config.cc $(HDRS)
	@mkdir -p build/san
	$(SAN_CXX) $(SAN_FLAGS) -fsanitize=address,undefined -fno-sanitize-recover=undefined -o $@ csrc/tests/fuzz_value.cc csrc/common/value.cc csrc/common/log.cc csrc/daemon/config.cc $(LDLIBS)

SAN_FUZZP_SRCS := $(sort $(HOST_SRCS) $(SHIM_SRCS)) csrc/tests/no_cuda_backend.cc csrc/tests/fuzz_protocol.cc
build/san/fuzz_protocol: $(SAN_FUZZP_SRCS) $(HDRS)
	@mkdir -p build/san
	$(SAN_CXX) $(SAN_FLAGS) -fsanitize=address,undefined -fno-sanitize-recover=undefined -o $@ $(SAN_FUZZP_SRCS) $(LDLIBS)

asan: build/san/stress_asan build/san/fuzz_value build/san/fuzz_protocol
	ASAN_OPTIONS="detect_leaks=1" build/san/stress_asan 40
	ASAN_OPTIONS="detect_leaks=1" build/san/stress_asan 40 memops
	build/san/fuzz_value 40000
	ASAN_OPTIONS="detect_leaks=1" build/san/fuzz_protocol 3000
	ASAN_OPTIONS="detect_leaks=1" build/san/fuzz_protocol 2000 client

# ---------------------------------------------------------------------------------------
# Evaluation recipes, one per figure of the reference's justfile (its `four_gpu_*`,
# `batched-allreduce-multi-final`, `run-dynamic` / `reconfig-ring`, `collect-setup4-*`
# recipes). They need the GPUs of one box; OUT collects the results.
# ---------------------------------------------------------------------------------------
NGPU ?= 8
OUT_DIR ?= out
PY ?= python
TORCHRUN = $(PY) -m torch.distributed.run --nnodes=1 --nproc-per-node $(NGPU) --master-addr 127.0.0.1

eval-single: all        # bandwidth vs. size for every variant, next to NCCL; table with roofline fractions
	@mkdir -p $(OUT_DIR)
	$(TORCHRUN) --master-port 29601 -m mccs_b200.utils.sweep --mode final --out $(OUT_DIR)/sweep_$(NGPU).csv
	$(PY) -m mccs_b200.utils.report $(OUT_DIR)/sweep_$(NGPU).csv > $(OUT_DIR)/sweep_$(NGPU).md

eval-tune: all          # measures a tuning table and merges it into configs/tuning_b200.json
	@mkdir -p $(OUT_DIR)
	$(TORCHRUN) --master-port 29602 -m mccs_b200.utils.sweep --mode tune --dtypes bf16 --out $(OUT_DIR)/tune_$(NGPU).csv \
	    --tuning $(OUT_DIR)/tuning_$(NGPU).json --merge-into configs/tuning_b200.json

eval-multi: all         # four co-located tenants under QoS weights, without the arbiter, and as independent NCCL groups; the reference's settings 1-4
	@mkdir -p $(OUT_DIR)
	$(PY) -m mccs_b200.utils.multi_tenant --iters 1000 > $(OUT_DIR)/multi_mccs.json
	$(PY) -m mccs_b200.utils.multi_tenant --iters 1000 --reconfig-at -1 --no-qos > $(OUT_DIR)/multi_mccs_noqos.json
	$(PY) -m mccs_b200.utils.multi_tenant --iters 1000 --backend nccl > $(OUT_DIR)/multi_nccl.json
	for s in 1 2 3 4; do \
	  $(PY) -m mccs_b200.utils.multi_tenant --setting $$s --batch 1 --bytes 134217728 --iters 300 --reconfig-at -1 > $(OUT_DIR)/setting$${s}_mccs.json; \
	  $(PY) -m mccs_b200.utils.multi_tenant --setting $$s --batch 1 --bytes 134217728 --iters 300 --backend nccl > $(OUT_DIR)/setting$${s}_nccl.json; \
	done

eval-dynamic: all       # a running job whose ring is reversed by the admin tool
	$(PY) -m mccs_b200.utils.launcher --benchmark configs/launch/reconfig.toml --output-dir $(OUT_DIR)

eval-traces: all        # the VGG + 2 x GPT traces side by side under fair / qosv1 / qosv2: job completion times
	@mkdir -p $(OUT_DIR)
	$(PY) -m mccs_b200.utils.colocate_traces --scale 1.0 --out $(OUT_DIR)/jct.json

eval-colocate: all      # ResNet-50 next to VGG-16; GPT-2-medium alone and with a ResNet-50 neighbour; service and NCCL
	@mkdir -p $(OUT_DIR)
	for sc in cnn gpt gpt-with-resnet; do for be in mccs nccl; do \
	  $(PY) -m mccs_b200.utils.colocate_train --scenario $$sc --backend $$be > $(OUT_DIR)/colocate_$${sc}_$$be.json; \
	done; done

eval-latency: all       # where the time of a small collective goes
	$(TORCHRUN) --master-port 29603 -m mccs_b200.utils.latency --bytes 64K

clean:
	rm -rf build $(OUT)/*.so $(OUT)/mccsd $(APP_BINS) $(OUT)/host_tests

.PHONY: all clean simtest tsan asan eval-single eval-tune eval-multi eval-dynamic eval-traces eval-colocate eval-latency
.SECONDARY:
