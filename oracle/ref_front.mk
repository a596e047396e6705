# Builds the reference's own C front half of MATMUL into oracle/_ref/ (test infrastructure).
#
#   make -f oracle/ref_front.mk REF=/path/to/open64        (REF: root of the reference tree; a default is set below)
#
# Compiled from the reference tree where it lies, nothing is copied:
#   osprey/libfi/matrix/matmul_<a><b>.c     the 80 _MATMUL_<A><B> wrappers whose strided kernels the
#                                           engine exports (_premult of matmul.h + the kernel call)
#   osprey/libfi/matrix/MATMUL_*dispatch.c  the 16 rank dispatchers in front of the BLAS hook
#   osprey/libfi/matrix/mmx_dlutil.c        the dlsym("sgemm_" ...) hook behind F90_MATMUL_BLAS
#   osprey/libfi/matrix/f90_mmult_error.c
#   osprey/libfi/dotprod/predot@.c          _PREDOT, the dope-vector parser of DOT_PRODUCT (as ref_PREDOT)
# Every reference entry point is renamed on the command line (-D_MATMUL_S4S4=ref_MATMUL_S4S4 for the
# wrappers, refdisp_MATMUL_S4S4 for the dispatchers) so that it can live in one process with the
# engine's entry point of the same name.  The arithmetic kernels of the reference are Fortran
# (s4gemmx.f ...) and no Fortran compiler exists here, so the wrappers' kernel calls are bound to
#   libfi_front_oracle.so   the CPU oracle's restatements (ref_front_xiface.c -> libo64ref.so)
#   libfi_front_engine.so   the engine's Fortran-ABI kernels in libo64gemm.so (needs a B200 to run)
REF     ?= /root/reference
HERE    := $(dir $(abspath $(lastword $(MAKEFILE_LIST))))
OUT     := $(HERE)_ref
SRC     := $(REF)/osprey/libfi/matrix
ENGINE  := $(abspath $(HERE)../open64_b200)
CC      := gcc
# -w: the sources are K&R-era C (implicit declarations of the Fortran kernels)
CFLAGS  := -O1 -fPIC -w -std=gnu89 -D_LITTLE_ENDIAN -DKEY -I$(REF)/osprey/clibinc -I$(REF)/osprey/libfi/include -I$(SRC)

KINDS   := c4c c4c4 c4i1 c4i2 c4i4 c4j c4s c4s4 cc4 cc@ ci1 ci2 ci4 cj@ cs4 cs@ i1c i1c4 i1i1 i1i2 i1i4 i1j i1s \
           i1s4 i2c i2c4 i2i1 i2i2 i2i4 i2j i2s i2s4 i4c i4c4 i4i1 i4i2 i4i4 i4j i4s i4s4 jc4 jc@ ji1 ji2 ji4 jj@ \
           js4 js@ l1l l1l1 l1l2 l1l4 l2l l2l1 l2l2 l2l4 l4l l4l1 l4l2 l4l4 ll1 ll2 ll4 ll@ s4c s4c4 s4i1 s4i2 s4i4 \
           s4j s4s s4s4 sc4 sc@ si1 si2 si4 sj@ ss4 ss@
DISP    := C4C4 C4C C4S4 C4S CC4 CC CS4 CS S4C4 S4C S4S4 S4S SC4 SC SS4 SS

upper    = $(shell echo '$(subst @,,$(1))' | tr 'a-z' 'A-Z')
WRAP_O  := $(foreach k,$(KINDS),$(OUT)/obj/matmul_$(subst @,,$(k)).o)
DISP_O  := $(foreach d,$(DISP),$(OUT)/obj/disp_$(d).o)
MISC_O  := $(OUT)/obj/mmx_dlutil.o $(OUT)/obj/f90_mmult_error.o $(OUT)/obj/predot.o $(OUT)/obj/glue.o

all: $(OUT)/libfi_front_oracle.so $(OUT)/libfi_front_engine.so

$(OUT)/obj:
	mkdir -p $@

define WRAP_RULE
$(OUT)/obj/matmul_$(subst @,,$(1)).o: $(SRC)/matmul_$(1).c | $(OUT)/obj
	$(CC) $(CFLAGS) -D_MATMUL_$(call upper,$(1))=ref_MATMUL_$(call upper,$(1)) -c '$$<' -o $$@
endef
$(foreach k,$(KINDS),$(eval $(call WRAP_RULE,$(k))))

define DISP_RULE
$(OUT)/obj/disp_$(1).o: $(SRC)/MATMUL_$(1)dispatch.c | $(OUT)/obj
	$(CC) $(CFLAGS) -D_MATMUL_$(1)=refdisp_MATMUL_$(1) -c $$< -o $$@
endef
$(foreach d,$(DISP),$(eval $(call DISP_RULE,$(d))))

$(OUT)/obj/mmx_dlutil.o: $(SRC)/mmx_dlutil.c | $(OUT)/obj
	$(CC) $(CFLAGS) -c $< -o $@
$(OUT)/obj/f90_mmult_error.o: $(SRC)/f90_mmult_error.c | $(OUT)/obj
	$(CC) $(CFLAGS) -c $< -o $@
$(OUT)/obj/predot.o: $(REF)/osprey/libfi/dotprod/predot@.c | $(OUT)/obj
	$(CC) $(CFLAGS) -D_PREDOT=ref_PREDOT -c '$<' -o $@
$(OUT)/obj/glue.o: $(HERE)ref_front_glue.c | $(OUT)/obj
	$(CC) -O1 -fPIC -Wall -std=gnu11 -ffp-contract=off -D_LITTLE_ENDIAN -DKEY -I$(REF)/osprey/clibinc -c $< -o $@
$(OUT)/obj/xiface.o: $(HERE)ref_front_xiface.c | $(OUT)/obj
	$(CC) -O1 -fPIC -Wall -std=gnu11 -c $< -o $@

$(HERE)libo64ref.so: $(HERE)gemm_ref.c
	$(MAKE) -C $(HERE) -f Makefile

$(OUT)/libfi_front_oracle.so: $(WRAP_O) $(DISP_O) $(MISC_O) $(OUT)/obj/xiface.o $(HERE)libo64ref.so
	$(CC) -shared -o $@ $(WRAP_O) $(DISP_O) $(MISC_O) $(OUT)/obj/xiface.o -L$(HERE) -lo64ref -ldl -Wl,-rpath,'$$ORIGIN/..' -Wl,-z,defs

$(OUT)/libfi_front_engine.so: $(WRAP_O) $(DISP_O) $(MISC_O) $(ENGINE)/libo64gemm.so
	$(CC) -shared -o $@ $(WRAP_O) $(DISP_O) $(MISC_O) -L$(ENGINE) -lo64gemm -ldl -Wl,-rpath,'$$ORIGIN/../../open64_b200' -Wl,-z,defs

clean:
	rm -rf $(OUT)/obj $(OUT)/libfi_front_oracle.so $(OUT)/libfi_front_engine.so

.PHONY: all clean
