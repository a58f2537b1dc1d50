"""The planning half of the one-call block (csrc/block_runner.cu) needs no GPU: asked for a plan only,
it chooses routes and sizes and launches nothing.  Its choice for the block's output (bfloat16 rows, or
float32 K slices that the next norm adds) has to be the one ``ops.linear`` makes from the same
thresholds, at every row count and at the widths of the real configurations; thresholds changed in
``ops`` have to reach it; a shape that no tensor-core kernel takes has to be refused, not guessed."""
import ctypes

import pytest
import torch

from coheryn_ai_studio_b200 import ops
from coheryn_ai_studio_b200.parts import native_block as nb

WIDTHS = {   # hidden, heads, kv heads, head size, intermediate
    "0.5b": (896, 14, 2, 64, 4864), "1.5b": (1536, 12, 2, 128, 8960), "7b": (3584, 28, 4, 128, 18944),
    "14b": (5120, 40, 8, 128, 13824)}


class Operand:
    """What the predicates of ops.py look at in a tensor."""

    def __init__(self, rows, cols):
        self.shape, self.dtype = (rows, cols), torch.bfloat16

    def stride(self, i):
        return self.shape[1] if i == 0 else 1

    def data_ptr(self):
        return 1 << 20

    def numel(self):
        return self.shape[0] * self.shape[1]

    def is_contiguous(self):
        return True


# A plan calls one function of the attention library, the one that sizes its scratch area; this stands in
# for it (so the test needs the core library only), and its address for the two entry points a plan never calls.
@ctypes.CFUNCTYPE(ctypes.c_long, ctypes.c_int, ctypes.c_int, ctypes.c_int)
def scratch_floats(B, nkv, max_kv_len):
    return B * nkv * ((max_kv_len + 127) // 128 + 1) * 160


def plan(width, T, B, q_len, max_kv_len, partial=True, shortest=None):
    H, nh, nkv, hd, I = WIDTHS[width] if isinstance(width, str) else width
    f = ctypes.cast(scratch_floats, ctypes.c_void_p).value
    a = 1 << 20     # a plan reads no memory: any aligned address stands for a tensor
    layer = nb.CoBlockLayer(a, a, a, a, a, None, a, a, a, f, f, f, 1e-6, 1e-6, hd ** -0.5, ops.BF16, ops.BF16, ops.BF16, ops.F32,
                            H, nh, nkv, hd, I, hd, 0, 1, 1 if partial else 0, 1 if partial else 0)
    step = nb.CoBlockStep(a, a, a, a, None, T, B, shortest or q_len, q_len, max_kv_len, 1)
    tuning = nb.CoBlockTuning(ops.SMALL_WEIGHT_ELEMENTS, ops.FEW_LARGE_WEIGHT, ops.ATTN_OPROJ_MERGE_BYTES, ops.FEW_M,
                              ops.FEW_DEFER_M, ops.FEW_HEAD_M, ops.SMALL_M, ops.SMALL_M_SHORT, ops.DEFER_MIN_K,
                              ops.DEFER_MIN_K_WIDE, ops.QKV_ROPE_M, ops.QKV_PARTS_M, ops.QKV_PARTS_FEW_FROM, ops.ATTN_OPROJ_M)
    out = nb.CoBlockPlan()
    rc = nb._entry_point()(ctypes.addressof(layer), ctypes.addressof(step), ctypes.addressof(tuning), a, a, 64, 16, a, 8, a, a, None,
                           0, 0, None, 0, 0, None, 0, 1, ctypes.addressof(out))
    plan.last = out
    return rc, out.out_kind, out.out_splits, out.scratch_bytes


FEW, FEW_DEFER, SMALL, MANY = 1, 2, 3, 4     # the products' routes as the plan numbers them


def linear_route(M, N, K, partial):
    """The if-chain of ops.linear over ops.py's own predicates."""
    x, w = Operand(M, K), Operand(N, K)
    if (partial and K >= (ops.DEFER_MIN_K_WIDE if M > ops.SMALL_M_SHORT else ops.DEFER_MIN_K)
            and ops._few_shape_ok(x, w, ops.FEW_DEFER_M) and ops.few_splits(N, K) > 1):
        return FEW_DEFER
    return FEW if ops._few_ok(x, w) else SMALL if ops._small_ok(x, w) else MANY if ops._tc_ok(x, w) else 0


class StepFacts:
    def __init__(self, B, q_len, max_kv_len):
        self.num_requests, self.max_q_len, self.max_kv_len = B, q_len, max_kv_len


def expected_routes(width, T, B, q_len, max_kv_len, partial):
    H, nh, nkv, hd, I = WIDTHS[width] if isinstance(width, str) else width
    Nq, Nqkv = nh * hd, (nh + 2 * nkv) * hd
    x, w_qkv, k_cache = Operand(T, H), Operand(Nqkv, H), Operand(1, 1)
    want = {}
    if ops.qkv_rope_ok(x, w_qkv, k_cache, hd, hd):
        want["qkv_route"] = 1
    else:
        count = ops.qkv_parts_count(x, w_qkv, k_cache, hd, hd)
        if count > 1:
            want["qkv_route"], want["qkv_parts"] = (2 if count == ops.few_splits(Nqkv, H) else 3), count
        else:
            want["qkv_route"], want["qkv_linear"] = 4, linear_route(T, Nqkv, H, False)
    merged = partial and ops.attention_oproj_ok(Operand(T, Nq), Operand(H, Nq), StepFacts(B, q_len, max_kv_len), nh, nkv, hd)
    want["merged"] = 1 if merged else 0
    if not merged:
        want["o_route"] = linear_route(T, H, Nq, partial)
    x2, w_gu = Operand(T, H), Operand(2 * I, H)
    want["gate_route"] = FEW if ops._few_ok(x2, w_gu) else SMALL if ops._small_ok(x2, w_gu) else MANY if ops._tc_ok(x2, w_gu) else 0
    want["down_route"] = linear_route(T, H, I, partial)
    return want


@pytest.mark.parametrize("width", sorted(WIDTHS))
def test_every_step_of_the_plan_goes_the_way_ops_would_send_it(width):
    cases = [(T, 1, T, T) for T in list(range(1, 140)) + [255, 256, 257, 300, 512, 2048]]     # a prompt portion
    cases += [(T, T, 1, kv) for T in (1, 2, 8, 16, 17, 32, 64, 128) for kv in (500, 4096, 32768)]   # decoding together
    cases += [(40, 3, 1, 900), (70, 5, 1, 3000)]      # decoded tokens beside a portion (the shortest run is one token)
    for T, B, q_len, kv in cases:
        for partial in (True, False):
            longest = q_len if B in (1, T) else T - B + 1      # mixed: one request brings all the other tokens
            rc = plan(width, T, B, longest, kv, partial, shortest=q_len)[0]
            nb_plan = plan.last
            want = expected_routes(width, T, B, longest, kv, partial)
            assert rc == 0, (T, B, partial)
            got = {k: getattr(nb_plan, k) for k in want}
            assert got == want, (T, B, kv, partial)


def expected_output(T, H, I, partial):
    """The first branch of ops.linear for the down projection (x: [T, I], w: [H, I])."""
    x, w = Operand(T, I), Operand(H, I)
    if (partial and I >= (ops.DEFER_MIN_K_WIDE if T > ops.SMALL_M_SHORT else ops.DEFER_MIN_K)
            and ops._few_shape_ok(x, w, ops.FEW_DEFER_M) and ops.few_splits(H, I) > 1):
        return 2, ops.few_splits(H, I)
    return 1, 1


@pytest.mark.parametrize("width", sorted(WIDTHS))
def test_the_plan_gives_the_output_that_ops_linear_would(width):
    H, _, _, _, I = WIDTHS[width]
    for T in list(range(1, 140)) + [255, 256, 257, 511, 512, 1000, 2048]:
        for partial in (True, False):
            rc, kind, splits, scratch = plan(width, T, 1, T, T, partial)
            assert rc == 0, (T, partial)
            want = expected_output(T, H, I, partial)
            assert (kind, splits if kind == 2 else 1) == want, (T, partial)
            assert scratch >= T * (H + I) * 2
    # decoding together: as many requests as rows
    for T in (1, 4, 8, 16, 17, 64):
        rc, kind, splits, _ = plan(width, T, T, 1, 3000)
        assert rc == 0 and (kind, splits if kind == 2 else 1) == expected_output(T, H, I, True)


def test_thresholds_set_in_ops_reach_the_plan(monkeypatch):
    H, _, _, _, I = WIDTHS["1.5b"]
    assert plan("1.5b", 8, 8, 1, 2000)[1] == 2          # eight rows: the down projection leaves its K slices
    monkeypatch.setattr(ops, "FEW_DEFER_M", 0)
    assert plan("1.5b", 8, 8, 1, 2000)[1] == 1
    assert expected_output(8, H, I, True) == (1, 1)


def test_a_width_no_tensor_core_kernel_takes_is_refused():
    rc, *_ = plan((100, 5, 1, 16, 36), 40, 1, 40, 40)     # a width of 100: rows that are no multiple of 16 bytes
    assert rc == nb.UNSUPPORTED


def test_random_widths_and_row_counts_go_the_same_way():
    """Widths nobody tuned for: any hidden and intermediate size that is a multiple of 8, head sizes in
    steps of 16, any number of heads and groups; row counts around every threshold and at random."""
    import numpy as np
    rng = np.random.default_rng(11)
    for _ in range(250):
        hd = int(rng.choice([16, 32, 48, 64, 80, 96, 128, 192, 256]))
        nkv = int(rng.integers(1, 9))
        nh = nkv * int(rng.integers(1, 9))
        width = (8 * int(rng.integers(8, 1025)), nh, nkv, hd, 8 * int(rng.integers(8, 3001)))
        rows = [1, 16, 17, 32, 33, 64, 65, 128, 129, 256, 257] + [int(t) for t in rng.integers(1, 3000, 4)]
        for T in rows:
            partial = bool(rng.integers(0, 2))
            if rng.integers(0, 2):
                B, longest, shortest, kv = 1, T, T, T + int(rng.integers(0, 5000))          # a portion
            else:
                B, longest, shortest, kv = T, 1, 1, int(rng.integers(1, 40000))             # decoding together
            rc = plan(width, T, B, longest, kv, partial, shortest=shortest)[0]
            assert rc == 0, (width, T)
            want = expected_routes(width, T, B, longest, kv, partial)
            got = {k: getattr(plan.last, k) for k in want}
            assert got == want, (width, T, B, kv, partial)
