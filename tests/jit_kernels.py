"""@triton.jit kernels used by the Triton-backend tests: K loops the backend must accept, in the shapes
users write them, and near misses it must refuse. Triton reads kernel source from a file, hence a module."""
import triton
import triton.language as tl


@triton.jit
def split_kloop(a_ptr, b_ptr, c_ptr, M, N, K, stride_am, stride_ak, stride_bk, stride_bn, stride_cm, stride_cn,
                K_MAIN, BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """The loop LoopSplit takes: the induction variable counts K elements and is compared with a
    loop-invariant split point; unmasked loads below it, masked loads from it on."""
    pid_m = tl.program_id(0)
    pid_n = tl.program_id(1)
    offs_m = pid_m * BLOCK_M + tl.arange(0, BLOCK_M)
    offs_n = pid_n * BLOCK_N + tl.arange(0, BLOCK_N)
    offs_k = tl.arange(0, BLOCK_K)
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, BLOCK_K):
        a_ptrs = a_ptr + offs_m[:, None] * stride_am + (k + offs_k)[None, :] * stride_ak
        b_ptrs = b_ptr + (k + offs_k)[:, None] * stride_bk + offs_n[None, :] * stride_bn
        if k < K_MAIN:
            a = tl.load(a_ptrs)
            b = tl.load(b_ptrs)
        else:
            a = tl.load(a_ptrs, mask=(k + offs_k)[None, :] < K, other=0.0)
            b = tl.load(b_ptrs, mask=(k + offs_k)[:, None] < K, other=0.0)
        acc = tl.dot(a, b, acc)
    c_ptrs = c_ptr + offs_m[:, None] * stride_cm + offs_n[None, :] * stride_cn
    tl.store(c_ptrs, acc.to(c_ptr.dtype.element_ty))


@triton.jit
def grouped_masked_kloop(a_ptr, b_ptr, c_ptr, M, N, K, stride_am, stride_ak, stride_bk, stride_bn, stride_cm,
                         stride_cn, alpha, BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr,
                         GROUP: tl.constexpr):
    """One-dimensional grid walked in groups of GROUP row tiles, a loop that counts K blocks, pointers
    advanced by the loop, every load masked on all three bounds, a scalar scale before the cast."""
    pid = tl.program_id(0)
    tiles_m = tl.cdiv(M, BLOCK_M)
    tiles_n = tl.cdiv(N, BLOCK_N)
    per_group = GROUP * tiles_n
    first_m = (pid // per_group) * GROUP
    rows_here = min(tiles_m - first_m, GROUP)
    pid_m = first_m + (pid % per_group) % rows_here
    pid_n = (pid % per_group) // rows_here
    rm = pid_m * BLOCK_M + tl.arange(0, BLOCK_M)
    rn = pid_n * BLOCK_N + tl.arange(0, BLOCK_N)
    rk = tl.arange(0, BLOCK_K)
    a_ptrs = a_ptr + rm[:, None] * stride_am + rk[None, :] * stride_ak
    b_ptrs = b_ptr + rk[:, None] * stride_bk + rn[None, :] * stride_bn
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for kb in range(0, tl.cdiv(K, BLOCK_K)):
        left = K - kb * BLOCK_K
        a = tl.load(a_ptrs, mask=(rm[:, None] < M) & (rk[None, :] < left), other=0.0)
        b = tl.load(b_ptrs, mask=(rk[:, None] < left) & (rn[None, :] < N), other=0.0)
        acc = tl.dot(a, b, acc)
        a_ptrs += BLOCK_K * stride_ak
        b_ptrs += BLOCK_K * stride_bk
    out = (acc * alpha).to(c_ptr.dtype.element_ty)
    c_ptrs = c_ptr + rm[:, None] * stride_cm + rn[None, :] * stride_cn
    tl.store(c_ptrs, out, mask=(rm[:, None] < M) & (rn[None, :] < N))


@triton.jit
def plain_kloop(a_ptr, b_ptr, c_ptr, K, stride_am, stride_ak, stride_bk, stride_bn, stride_cm,
                BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """No masks at all: every extent is a multiple of its block."""
    rm = tl.program_id(1) * BLOCK_M + tl.arange(0, BLOCK_M)
    rn = tl.program_id(0) * BLOCK_N + tl.arange(0, BLOCK_N)
    rk = tl.arange(0, BLOCK_K)
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, BLOCK_K):
        a = tl.load(a_ptr + rm[:, None] * stride_am + (k + rk)[None, :] * stride_ak)
        b = tl.load(b_ptr + (k + rk)[:, None] * stride_bk + rn[None, :] * stride_bn)
        acc += tl.dot(a, b)
    tl.store(c_ptr + rm[:, None] * stride_cm + rn[None, :], acc.to(c_ptr.dtype.element_ty))


@triton.jit
def relu_kloop(a_ptr, b_ptr, c_ptr, K, stride_am, stride_bk, stride_cm,
               BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """Near miss: an activation between the loop and the store."""
    rm = tl.program_id(0) * BLOCK_M + tl.arange(0, BLOCK_M)
    rn = tl.program_id(1) * BLOCK_N + tl.arange(0, BLOCK_N)
    rk = tl.arange(0, BLOCK_K)
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, BLOCK_K):
        a = tl.load(a_ptr + rm[:, None] * stride_am + (k + rk)[None, :])
        b = tl.load(b_ptr + (k + rk)[:, None] * stride_bk + rn[None, :])
        acc = tl.dot(a, b, acc)
    acc = tl.maximum(acc, 0.0)
    tl.store(c_ptr + rm[:, None] * stride_cm + rn[None, :], acc.to(c_ptr.dtype.element_ty))


@triton.jit
def shifted_rows_kloop(a_ptr, b_ptr, c_ptr, K, stride_am, stride_bk, stride_cm,
                       BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """A is read one row further down than C is written: the product of A without its first row."""
    rm = tl.program_id(0) * BLOCK_M + tl.arange(0, BLOCK_M)
    rn = tl.program_id(1) * BLOCK_N + tl.arange(0, BLOCK_N)
    rk = tl.arange(0, BLOCK_K)
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, BLOCK_K):
        a = tl.load(a_ptr + (rm + 1)[:, None] * stride_am + (k + rk)[None, :])
        b = tl.load(b_ptr + (k + rk)[:, None] * stride_bk + rn[None, :])
        acc = tl.dot(a, b, acc)
    tl.store(c_ptr + rm[:, None] * stride_cm + rn[None, :], acc.to(c_ptr.dtype.element_ty))


@triton.jit
def strided_k_kloop(a_ptr, b_ptr, c_ptr, K, stride_am, stride_bk, stride_cm,
                    BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """Near miss: the loop skips every other K block."""
    rm = tl.program_id(0) * BLOCK_M + tl.arange(0, BLOCK_M)
    rn = tl.program_id(1) * BLOCK_N + tl.arange(0, BLOCK_N)
    rk = tl.arange(0, BLOCK_K)
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, 2 * BLOCK_K):
        a = tl.load(a_ptr + rm[:, None] * stride_am + (k + rk)[None, :])
        b = tl.load(b_ptr + (k + rk)[:, None] * stride_bk + rn[None, :])
        acc = tl.dot(a, b, acc)
    tl.store(c_ptr + rm[:, None] * stride_cm + rn[None, :], acc.to(c_ptr.dtype.element_ty))


@triton.jit
def nonzero_fill_kloop(a_ptr, b_ptr, c_ptr, K, stride_am, stride_bk, stride_cm,
                       BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """Near miss: masked-off K elements read as one, not zero."""
    rm = tl.program_id(0) * BLOCK_M + tl.arange(0, BLOCK_M)
    rn = tl.program_id(1) * BLOCK_N + tl.arange(0, BLOCK_N)
    rk = tl.arange(0, BLOCK_K)
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, BLOCK_K):
        a = tl.load(a_ptr + rm[:, None] * stride_am + (k + rk)[None, :], mask=(k + rk)[None, :] < K, other=1.0)
        b = tl.load(b_ptr + (k + rk)[:, None] * stride_bk + rn[None, :], mask=(k + rk)[:, None] < K, other=0.0)
        acc = tl.dot(a, b, acc)
    tl.store(c_ptr + rm[:, None] * stride_cm + rn[None, :], acc.to(c_ptr.dtype.element_ty))


@triton.jit
def scaled_kloop(a_ptr, b_ptr, c_ptr, rs_ptr, cs_ptr, M, N, K, stride_am, stride_bk, stride_cm, alpha,
                 BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """The quantised-GEMM epilogue: per-row and per-column fp32 factors and a scalar, then the cast."""
    rm = tl.program_id(0) * BLOCK_M + tl.arange(0, BLOCK_M)
    rn = tl.program_id(1) * BLOCK_N + tl.arange(0, BLOCK_N)
    rk = tl.arange(0, BLOCK_K)
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, BLOCK_K):
        a = tl.load(a_ptr + rm[:, None] * stride_am + (k + rk)[None, :],
                    mask=(rm[:, None] < M) & ((k + rk)[None, :] < K), other=0.0)
        b = tl.load(b_ptr + (k + rk)[:, None] * stride_bk + rn[None, :],
                    mask=((k + rk)[:, None] < K) & (rn[None, :] < N), other=0.0)
        acc = tl.dot(a, b, acc)
    rs = tl.load(rs_ptr + rm, mask=rm < M, other=0.0)
    cs = tl.load(cs_ptr + rn, mask=rn < N, other=0.0)
    out = acc * rs[:, None] * cs[None, :] * alpha
    tl.store(c_ptr + rm[:, None] * stride_cm + rn[None, :], out.to(c_ptr.dtype.element_ty),
             mask=(rm[:, None] < M) & (rn[None, :] < N))


@triton.jit
def wrong_scale_kloop(a_ptr, b_ptr, c_ptr, rs_ptr, K, stride_am, stride_bk, stride_cm,
                      BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """Near miss: the row factors are read from the next tile's rows."""
    rm = tl.program_id(0) * BLOCK_M + tl.arange(0, BLOCK_M)
    rn = tl.program_id(1) * BLOCK_N + tl.arange(0, BLOCK_N)
    rk = tl.arange(0, BLOCK_K)
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, BLOCK_K):
        a = tl.load(a_ptr + rm[:, None] * stride_am + (k + rk)[None, :])
        b = tl.load(b_ptr + (k + rk)[:, None] * stride_bk + rn[None, :])
        acc = tl.dot(a, b, acc)
    rs = tl.load(rs_ptr + rm + BLOCK_M)
    tl.store(c_ptr + rm[:, None] * stride_cm + rn[None, :], (acc * rs[:, None]).to(c_ptr.dtype.element_ty))


@triton.jit
def wrapped_kloop(a_ptr, b_ptr, c_ptr, M, N, K, stride_am, stride_ak, stride_bk, stride_bn, stride_cm, stride_cn,
                  BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """Row and column indices of the loads wrap around the matrix instead of being masked; only K is masked
    in the loop and only the store masks rows and columns. Compiler hints on the indices."""
    pid = tl.program_id(0)
    tiles_n = tl.cdiv(N, BLOCK_N)
    pid_m = pid // tiles_n
    pid_n = pid % tiles_n
    tl.assume(pid_m >= 0)
    tl.assume(stride_am > 0)
    rm = (pid_m * BLOCK_M + tl.arange(0, BLOCK_M)) % M
    rn = (pid_n * BLOCK_N + tl.arange(0, BLOCK_N)) % N
    rm = tl.max_contiguous(tl.multiple_of(rm, BLOCK_M), BLOCK_M)
    rk = tl.arange(0, BLOCK_K)
    a_ptrs = a_ptr + (rm[:, None] * stride_am + rk[None, :] * stride_ak)
    b_ptrs = b_ptr + (rk[:, None] * stride_bk + rn[None, :] * stride_bn)
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for kb in range(0, tl.cdiv(K, BLOCK_K)):
        a = tl.load(a_ptrs, mask=rk[None, :] < K - kb * BLOCK_K, other=0.0)
        b = tl.load(b_ptrs, mask=rk[:, None] < K - kb * BLOCK_K, other=0.0)
        acc = tl.dot(a, b, acc)
        a_ptrs += BLOCK_K * stride_ak
        b_ptrs += BLOCK_K * stride_bk
    cm = pid_m * BLOCK_M + tl.arange(0, BLOCK_M)
    cn = pid_n * BLOCK_N + tl.arange(0, BLOCK_N)
    tl.store(c_ptr + stride_cm * cm[:, None] + stride_cn * cn[None, :], acc.to(c_ptr.dtype.element_ty),
             mask=(cm[:, None] < M) & (cn[None, :] < N))


@triton.jit
def wrapped_unmasked_store_kloop(a_ptr, b_ptr, c_ptr, M, K, stride_am, stride_bk, stride_cm,
                                 BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """Near miss: rows wrap around M but the store keeps the wrapped rows."""
    rm = tl.program_id(0) * BLOCK_M + tl.arange(0, BLOCK_M)
    rn = tl.program_id(1) * BLOCK_N + tl.arange(0, BLOCK_N)
    rk = tl.arange(0, BLOCK_K)
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, BLOCK_K):
        a = tl.load(a_ptr + (rm % M)[:, None] * stride_am + (k + rk)[None, :])
        b = tl.load(b_ptr + (k + rk)[:, None] * stride_bk + rn[None, :])
        acc = tl.dot(a, b, acc)
    tl.store(c_ptr + rm[:, None] * stride_cm + rn[None, :], acc.to(c_ptr.dtype.element_ty))


@triton.jit
def _tile_of(t, tiles_m, tiles_n, GROUP: tl.constexpr):
    per_group = GROUP * tiles_n
    first_m = (t // per_group) * GROUP
    rows_here = min(tiles_m - first_m, GROUP)
    return first_m + (t % per_group) % rows_here, (t % per_group) // rows_here


@triton.jit
def persistent_kloop(a_ptr, b_ptr, c_ptr, M, N, K, stride_am, stride_bk, stride_cm,
                     BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr, GROUP: tl.constexpr):
    """A persistent kernel: as many programs as the launch gives, each walking the tiles of C with a stride
    of the program count; a helper function maps the tile number to a grouped (row, column) order."""
    tiles_m = tl.cdiv(M, BLOCK_M)
    tiles_n = tl.cdiv(N, BLOCK_N)
    rk = tl.arange(0, BLOCK_K)
    for t in range(tl.program_id(0), tiles_m * tiles_n, tl.num_programs(0)):
        pid_m, pid_n = _tile_of(t, tiles_m, tiles_n, GROUP)
        rm = pid_m * BLOCK_M + tl.arange(0, BLOCK_M)
        rn = pid_n * BLOCK_N + tl.arange(0, BLOCK_N)
        acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
        for k in range(0, K, BLOCK_K):
            a = tl.load(a_ptr + rm[:, None] * stride_am + (k + rk)[None, :],
                        mask=(rm[:, None] < M) & ((k + rk)[None, :] < K), other=0.0)
            b = tl.load(b_ptr + (k + rk)[:, None] * stride_bk + rn[None, :],
                        mask=((k + rk)[:, None] < K) & (rn[None, :] < N), other=0.0)
            acc = tl.dot(a, b, acc)
        tl.store(c_ptr + rm[:, None] * stride_cm + rn[None, :], acc.to(c_ptr.dtype.element_ty),
                 mask=(rm[:, None] < M) & (rn[None, :] < N))


@triton.jit
def descriptor_kloop(a_ptr, b_ptr, c_ptr, M, N, K, stride_am, stride_bk, stride_cm,
                     BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """Operands and result through in-kernel tensor descriptors: bounds come from the descriptor shapes."""
    a_desc = tl.make_tensor_descriptor(a_ptr, shape=[M, K], strides=[stride_am, 1], block_shape=[BLOCK_M, BLOCK_K])
    b_desc = tl.make_tensor_descriptor(b_ptr, shape=[K, N], strides=[stride_bk, 1], block_shape=[BLOCK_K, BLOCK_N])
    c_desc = tl.make_tensor_descriptor(c_ptr, shape=[M, N], strides=[stride_cm, 1], block_shape=[BLOCK_M, BLOCK_N])
    row = tl.program_id(0) * BLOCK_M
    col = tl.program_id(1) * BLOCK_N
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, BLOCK_K):
        a = a_desc.load([row, k])
        b = b_desc.load([k, col])
        acc = tl.dot(a, b, acc)
    c_desc.store([row, col], acc.to(c_ptr.dtype.element_ty))


@triton.jit
def nt_kloop(a_ptr, bt_ptr, c_ptr, M, N, K, stride_am, stride_bn, stride_cm,
             BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """C = A @ Bt^T with Bt stored [N, K]: the B tile is loaded as [BLOCK_N, BLOCK_K] and transposed in
    registers, the way the reference's attention feeds K to its first dot."""
    rm = tl.program_id(0) * BLOCK_M + tl.arange(0, BLOCK_M)
    rn = tl.program_id(1) * BLOCK_N + tl.arange(0, BLOCK_N)
    rk = tl.arange(0, BLOCK_K)
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, BLOCK_K):
        a = tl.load(a_ptr + rm[:, None] * stride_am + (k + rk)[None, :],
                    mask=(rm[:, None] < M) & ((k + rk)[None, :] < K), other=0.0)
        bt = tl.load(bt_ptr + rn[:, None] * stride_bn + (k + rk)[None, :],
                     mask=(rn[:, None] < N) & ((k + rk)[None, :] < K), other=0.0)
        acc = tl.dot(a, tl.trans(bt), acc)
    tl.store(c_ptr + rm[:, None] * stride_cm + rn[None, :], acc.to(c_ptr.dtype.element_ty),
             mask=(rm[:, None] < M) & (rn[None, :] < N))


@triton.jit
def narrowed_operand_kloop(a_ptr, b_ptr, c_ptr, K, stride_am, stride_bk, stride_cm,
                           BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """Near miss: the operands are rounded to fp8 between the load and the dot."""
    rm = tl.program_id(0) * BLOCK_M + tl.arange(0, BLOCK_M)
    rn = tl.program_id(1) * BLOCK_N + tl.arange(0, BLOCK_N)
    rk = tl.arange(0, BLOCK_K)
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, BLOCK_K):
        a = tl.load(a_ptr + rm[:, None] * stride_am + (k + rk)[None, :]).to(tl.float8e4nv)
        b = tl.load(b_ptr + (k + rk)[:, None] * stride_bk + rn[None, :]).to(tl.float8e4nv)
        acc = tl.dot(a, b, acc)
    tl.store(c_ptr + rm[:, None] * stride_cm + rn[None, :], acc.to(c_ptr.dtype.element_ty))


@triton.jit
def half_accumulator_kloop(a_ptr, b_ptr, c_ptr, K, stride_am, stride_bk, stride_cm,
                           BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """Near miss: the accumulator is fp16."""
    rm = tl.program_id(0) * BLOCK_M + tl.arange(0, BLOCK_M)
    rn = tl.program_id(1) * BLOCK_N + tl.arange(0, BLOCK_N)
    rk = tl.arange(0, BLOCK_K)
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float16)
    for k in range(0, K, BLOCK_K):
        a = tl.load(a_ptr + rm[:, None] * stride_am + (k + rk)[None, :])
        b = tl.load(b_ptr + (k + rk)[:, None] * stride_bk + rn[None, :])
        acc = tl.dot(a, b, acc, out_dtype=tl.float16)
    tl.store(c_ptr + rm[:, None] * stride_cm + rn[None, :], acc)


@triton.jit
def widened_operand_kloop(a_ptr, b_ptr, c_ptr, K, stride_am, stride_bk, stride_cm,
                          BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """bf16 operands widened to fp32 before the dot (exact), fp32 result: what the interpreter oracle's kernel does."""
    rm = tl.program_id(0) * BLOCK_M + tl.arange(0, BLOCK_M)
    rn = tl.program_id(1) * BLOCK_N + tl.arange(0, BLOCK_N)
    rk = tl.arange(0, BLOCK_K)
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, BLOCK_K):
        a = tl.load(a_ptr + rm[:, None] * stride_am + (k + rk)[None, :]).to(tl.float32)
        b = tl.load(b_ptr + (k + rk)[:, None] * stride_bk + rn[None, :]).to(tl.float32)
        acc = tl.dot(a, b, acc, input_precision="ieee")
    tl.store(c_ptr + rm[:, None] * stride_cm + rn[None, :], acc)


@triton.jit
def counting_kloop(a_ptr, b_ptr, c_ptr, count_ptr, K, stride_am, stride_bk, stride_cm,
                   BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """Near miss: a correct GEMM that also counts its programs with an atomic."""
    rm = tl.program_id(0) * BLOCK_M + tl.arange(0, BLOCK_M)
    rn = tl.program_id(1) * BLOCK_N + tl.arange(0, BLOCK_N)
    rk = tl.arange(0, BLOCK_K)
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, BLOCK_K):
        a = tl.load(a_ptr + rm[:, None] * stride_am + (k + rk)[None, :])
        b = tl.load(b_ptr + (k + rk)[:, None] * stride_bk + rn[None, :])
        acc = tl.dot(a, b, acc)
    tl.atomic_add(count_ptr, 1)
    tl.store(c_ptr + rm[:, None] * stride_cm + rn[None, :], acc.to(c_ptr.dtype.element_ty))


@triton.jit
def vector_add(x_ptr, y_ptr, out_ptr, n, BLOCK: tl.constexpr):
    """Not a GEMM at all."""
    offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
    mask = offs < n
    tl.store(out_ptr + offs, tl.load(x_ptr + offs, mask=mask) + tl.load(y_ptr + offs, mask=mask), mask=mask)


@triton.jit
def row_softmax(x_ptr, out_ptr, n_cols, stride, BLOCK: tl.constexpr):
    """Not a GEMM: a reduction (an operation with a region) and exponentials."""
    row = tl.program_id(0)
    offs = tl.arange(0, BLOCK)
    x = tl.load(x_ptr + row * stride + offs, mask=offs < n_cols, other=-float("inf"))
    e = tl.exp(x - tl.max(x, axis=0))
    tl.store(out_ptr + row * stride + offs, e / tl.sum(e, axis=0), mask=offs < n_cols)


@triton.jit
def two_dots_kloop(a_ptr, b_ptr, c_ptr, K, stride_am, stride_bk, stride_cm,
                   BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """Near miss: the product of A with B is multiplied by B's first tile again (two tt.dot)."""
    rm = tl.program_id(0) * BLOCK_M + tl.arange(0, BLOCK_M)
    rn = tl.program_id(1) * BLOCK_N + tl.arange(0, BLOCK_N)
    rk = tl.arange(0, BLOCK_K)
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, BLOCK_K):
        a = tl.load(a_ptr + rm[:, None] * stride_am + (k + rk)[None, :])
        b = tl.load(b_ptr + (k + rk)[:, None] * stride_bk + rn[None, :])
        acc = tl.dot(a, b, acc)
    w = tl.load(b_ptr + tl.arange(0, BLOCK_N)[:, None] * stride_bk + rn[None, :])
    out = tl.dot(acc.to(tl.bfloat16), w)
    tl.store(c_ptr + rm[:, None] * stride_cm + rn[None, :], out.to(c_ptr.dtype.element_ty))


@triton.jit
def batched_kloop(a_ptr, b_ptr, c_ptr, K, stride_ab, stride_am, stride_bb, stride_bk, stride_cb, stride_cm,
                  BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """One matrix product per program_id(2), each at its own base offset in A, B and C."""
    batch = tl.program_id(2)
    rm = tl.program_id(0) * BLOCK_M + tl.arange(0, BLOCK_M)
    rn = tl.program_id(1) * BLOCK_N + tl.arange(0, BLOCK_N)
    rk = tl.arange(0, BLOCK_K)
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, BLOCK_K):
        a = tl.load(a_ptr + batch * stride_ab + rm[:, None] * stride_am + (k + rk)[None, :])
        b = tl.load(b_ptr + batch * stride_bb + (k + rk)[:, None] * stride_bk + rn[None, :])
        acc = tl.dot(a, b, acc)
    tl.store(c_ptr + batch * stride_cb + rm[:, None] * stride_cm + rn[None, :], acc.to(c_ptr.dtype.element_ty))


@triton.jit
def block_pointer_kloop(a_ptr, b_ptr, c_ptr, M, N, K, stride_am, stride_bk, stride_cm,
                        BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """Operands through block pointers advanced by the loop, with boundary checks on both axes, as the
    reference's attention kernel addresses Q, K and V (tl.make_block_ptr / tl.advance)."""
    pid_m = tl.program_id(0)
    pid_n = tl.program_id(1)
    a_blk = tl.make_block_ptr(base=a_ptr, shape=(M, K), strides=(stride_am, 1), offsets=(pid_m * BLOCK_M, 0),
                              block_shape=(BLOCK_M, BLOCK_K), order=(1, 0))
    b_blk = tl.make_block_ptr(base=b_ptr, shape=(K, N), strides=(stride_bk, 1), offsets=(0, pid_n * BLOCK_N),
                              block_shape=(BLOCK_K, BLOCK_N), order=(1, 0))
    c_blk = tl.make_block_ptr(base=c_ptr, shape=(M, N), strides=(stride_cm, 1),
                              offsets=(pid_m * BLOCK_M, pid_n * BLOCK_N), block_shape=(BLOCK_M, BLOCK_N), order=(1, 0))
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, BLOCK_K):
        a = tl.load(a_blk, boundary_check=(0, 1), padding_option="zero")
        b = tl.load(b_blk, boundary_check=(0, 1), padding_option="zero")
        acc = tl.dot(a, b, acc)
        a_blk = tl.advance(a_blk, (0, BLOCK_K))
        b_blk = tl.advance(b_blk, (BLOCK_K, 0))
    tl.store(c_blk, acc.to(c_ptr.dtype.element_ty), boundary_check=(0, 1))


@triton.jit
def single_dot(a_ptr, b_ptr, c_ptr, M, N, K, stride_am, stride_bk, stride_cm,
               BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """No K loop: K fits one tile (masked against K), one tt.dot."""
    rm = tl.program_id(0) * BLOCK_M + tl.arange(0, BLOCK_M)
    rn = tl.program_id(1) * BLOCK_N + tl.arange(0, BLOCK_N)
    rk = tl.arange(0, BLOCK_K)
    a = tl.load(a_ptr + rm[:, None] * stride_am + rk[None, :], mask=(rm[:, None] < M) & (rk[None, :] < K), other=0.0)
    b = tl.load(b_ptr + rk[:, None] * stride_bk + rn[None, :], mask=(rk[:, None] < K) & (rn[None, :] < N), other=0.0)
    acc = tl.dot(a, b)
    tl.store(c_ptr + rm[:, None] * stride_cm + rn[None, :], acc.to(c_ptr.dtype.element_ty),
             mask=(rm[:, None] < M) & (rn[None, :] < N))


@triton.jit
def host_descriptor_kloop(a_desc, b_desc, c_desc, K, BLOCK_M: tl.constexpr, BLOCK_N: tl.constexpr, BLOCK_K: tl.constexpr):
    """Operands and result as tensor descriptors built on the host and passed as arguments, the form of the
    reference's `_attn_fwd_tma`."""
    row = tl.program_id(0) * BLOCK_M
    col = tl.program_id(1) * BLOCK_N
    acc = tl.zeros((BLOCK_M, BLOCK_N), dtype=tl.float32)
    for k in range(0, K, BLOCK_K):
        a = a_desc.load([row, k])
        b = b_desc.load([k, col])
        acc = tl.dot(a, b, acc)
    c_desc.store([row, col], acc.to(c_desc.dtype))
