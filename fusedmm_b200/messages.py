"""The ``imessage`` wire format of ``fusedMM_csr`` (HipGraph/FusedMM ``fusedMM.h:18-73``): five 4-bit stage
codes, VOP in bits 0-3, ROP 4-7, SOP 8-11, VSC (MOP) 12-15, AOP 16-19."""

VOP_NOOP, VOP_COPY_LHS, VOP_COPY_RHS, VOP_ADD, VOP_SUBL, VOP_SUBR, VOP_MAX, VOP_MIN, VOP_UDEF = (
    0x0, 0x1, 0x2, 0x3, 0x4, 0x5, 0x6, 0x7, 0xF)
ROP_NOOP, ROP_DOT, ROP_ADD_LHS, ROP_ADD_RHS, ROP_NORML, ROP_NORMR, ROP_UDEF = (
    0x00, 0x10, 0x20, 0x30, 0x40, 0x50, 0xF0)
SOP_NOOP, SOP_COPY, SOP_UDEF = 0x000, 0x100, 0xF00
VSC_NOOP, VSC_MUL, VSC_ADD, VSC_UDEF = 0x0000, 0x1000, 0x2000, 0xF000
AOP_NOOP, AOP_ADD, AOP_MAX, AOP_MIN, AOP_UDEF = 0x00000, 0x10000, 0x20000, 0x30000, 0xF0000

# The four messages the reference has optimised kernels for (fusedMM.c:523-594) and the letters its
# dispatcher uses for them (kernels/src/kernels.c:456-631).
MSG_SIGMOID = VOP_COPY_RHS | ROP_DOT | SOP_UDEF | VSC_MUL | AOP_ADD      # 's'  0x11F12
MSG_TDIST = VOP_SUBR | ROP_NORMR | SOP_UDEF | VSC_MUL | AOP_ADD          # 't' (and FR)  0x11F55
MSG_SPMM = VOP_COPY_RHS | ROP_NOOP | SOP_COPY | VSC_MUL | AOP_ADD        # 'm'  0x11102
MSG_GCN = VOP_COPY_RHS | ROP_NOOP | SOP_NOOP | VSC_NOOP | AOP_ADD        # 'g'  0x10002

# Scalar functions SOP_UDEF can stand for on the device (include/fusedmm_b200.h).
SOP_IDENTITY, SOP_SIGMOID, SOP_SIGMOID_TABLE_C, SOP_FR, SOP_TDIST, SOP_TDIST_CLAMPED, SOP_LL, SOP_FA, \
    SOP_AFFINE_RECIP = range(9)

# Status codes (fusedMM.h:103-112 plus the CUDA-side additions of include/fusedmm_b200.h).
OK, ERR_VOP, ERR_ROP, ERR_AOP, ERR_SOP, ERR_VSC, ERR_UDEF, ERR_NO_OPT = 0, 2, 4, 8, 16, 32, 64, 128
ERR_NOMEM, ERR_CUDA, ERR_ARG, ERR_LIMIT = -1, -2, -3, -4

# flops per edge and per feature used for GFLOP/s, the reference's own accounting
# (test/fusedMMtime.cpp:816-828)
FLOPS_PER_EDGE_PER_K = {MSG_SIGMOID: 4, MSG_TDIST: 5, MSG_SPMM: 2, MSG_GCN: 1}


def message(vop, rop, sop, vsc, aop):
    return vop | rop | sop | vsc | aop
