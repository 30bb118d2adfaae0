"""CPU-side checks of the C ABI: the library loads, exports every symbol the header declares,
and the host mirror validates arguments like the reference does. No compute call is made."""
import os
import re

import pytest

from helpers import ROOT, pkg


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "darkforest_kernels.h")).read()
    return re.findall(r"^DF_API\s+[\w\s\*]+?\b(\w+)\(", text, flags=re.M)


def test_library_loads_and_exports_every_declared_symbol():
    p = pkg()
    if not os.path.exists(p.LIB_PATH):
        p.build()
    L = p.lib()
    names = _header_symbols()
    assert len(names) >= 19
    for n in names:
        assert hasattr(L, n), n
        assert n in p.PROTOTYPES, f"{n} declared in the header but not bound"
    assert set(p.PROTOTYPES) == set(names)
    for legacy in ("launch_fused_attention", "launch_fused_mha_forward", "launch_attention_backward",
                   "launch_fused_mha_backward", "darkforest_sync"):
        assert legacy in names
    assert b"sm_100a" in L.df_attn_build_info()


def test_status_strings_and_variant_switch():
    p = pkg()
    L = p.lib()
    assert L.df_attn_status_string(p.DF_OK) == b"ok"
    for code in (p.DF_ERR_INVALID_ARG, p.DF_ERR_UNSUPPORTED, p.DF_ERR_CUDA, p.DF_ERR_DEVICE_TIMEOUT,
                 p.DF_ERR_WORKSPACE):
        assert L.df_attn_status_string(code) not in (b"ok", b"unknown status")
    prev = p.set_variant(p.VARIANT_SIMT)
    assert p.set_variant(prev) == p.VARIANT_SIMT
    assert p.set_variant(99) == prev and p.set_variant(prev) == prev  # out of range is ignored


def test_argument_validation_happens_on_the_host():
    p = pkg()
    L = p.lib()
    # D outside 1..128 and null pointers are rejected before any CUDA call
    assert L.df_attn_forward(None, None, None, None, None, 1, 1, 16, 0, 1.0, 1, None) == p.DF_ERR_INVALID_ARG
    assert L.df_attn_forward(None, None, None, None, None, 1, 1, 16, 129, 1.0, 1, None) == p.DF_ERR_INVALID_ARG
    assert L.df_attn_forward(None, None, None, None, None, 1, 1, 16, 64, 1.0, 1, None) == p.DF_ERR_INVALID_ARG
    assert L.df_attn_forward(None, None, None, None, None, 1, 0, 16, 64, 1.0, 1, None) == p.DF_ERR_INVALID_ARG
    # empty problems are no-ops
    assert L.df_attn_forward(None, None, None, None, None, 1, 4, 0, 64, 1.0, 1, None) == p.DF_OK
    assert L.df_attn_forward(None, None, None, None, None, 0, 4, 16, 64, 1.0, 1, None) == p.DF_OK
    # legacy void symbols record a sticky status instead of aborting
    L.df_attn_last_status()
    L.launch_fused_mha_forward(None, None, None, None, 4, 16, 200, 1.0, 1)
    assert L.df_attn_last_status() == p.DF_ERR_INVALID_ARG
    assert L.df_attn_last_status() == p.DF_OK


def test_attention_context_mirrors_reference_checks():
    p = pkg()
    with pytest.raises(p.AttentionError):
        p.AttentionContext(12, 128, 0)
    with pytest.raises(p.AttentionError):
        p.AttentionContext(12, 128, 129)
    ctx = p.AttentionContext(12, 128, 64)
    assert ctx.d_model == 768
    import torch
    cpu = torch.zeros(128, 768)
    with pytest.raises(p.AttentionError):  # no CPU path
        ctx.forward_device_into(cpu, cpu, cpu, 0.125, True, cpu)
    with pytest.raises(p.AttentionError):  # shape mismatch, lib.rs:2051
        ctx.forward_device_into(cpu, cpu, cpu, 0.125, True, torch.zeros(64, 768))


def test_persistent_schedule_covers_every_item_once_and_balances_the_causal_triangle():
    """df_attn_schedule_item is the function the persistent kernels use to pick their work: every item must be
    taken exactly once, each CTA's list must be contiguous in rounds, and on causal workloads (items numbered
    heaviest first) the heaviest CTA must stay close to the average load."""
    import heapq
    L = pkg().lib()

    def lists(n_items, grid):
        out = []
        for cta in range(grid):
            mine, ended = [], False
            for r in range(n_items // grid + 3):
                idx = L.df_attn_schedule_item(r, grid, cta, n_items)
                if idx < 0:
                    ended = True
                else:
                    assert not ended, "a CTA's list has a hole"
                    mine.append(idx)
            out.append(mine)
        return out

    for n_items, grid in [(1, 1), (5, 148), (148, 148), (149, 148), (384, 148), (768, 148), (1000, 7)]:
        got = sorted(i for l in lists(n_items, grid) for i in l)
        assert got == list(range(n_items)), (n_items, grid)
    assert L.df_attn_schedule_item(0, 148, 148, 10) == -1 and L.df_attn_schedule_item(-1, 148, 0, 10) == -1

    def lpt(weights, grid):
        h = [0] * grid
        heapq.heapify(h)
        for w in weights:
            heapq.heappush(h, heapq.heappop(h) + w)
        return max(h)

    # forward: pairs of query tiles of B*H heads, weight = key tiles of the later tile; backward: key tiles
    cases = {"fwd S=1024 B*H=96": [2 * (4 - p) for p in range(4) for _ in range(96)],
             "fwd S=32768 B*H=12": [2 * (128 - p) for p in range(128) for _ in range(12)],
             "bwd S=1024 B*H=96": [8 - k for k in range(8) for _ in range(96)],
             "bwd S=16384 B*H=12": [128 - k for k in range(128) for _ in range(12)]}
    for name, w in cases.items():
        loads = [sum(w[i] for i in l) for l in lists(len(w), 148)]
        assert max(loads) <= lpt(w, 148) * 1.01 + 1e-9, (name, max(loads), lpt(w, 148))
        assert max(loads) <= 1.09 * sum(w) / 148, (name, max(loads), sum(w) / 148)


def test_workspace_sizes():
    L = pkg().lib()
    B, H, S, D = 8, 12, 1024, 64
    assert L.df_attn_workspace_bytes(0, B, H, S, D, 0) == B * H * S * 4
    assert L.df_attn_workspace_bytes(1, B, H, S, D, 0) == B * H * S * 4
    assert L.df_attn_workspace_bytes(2, 1, H, S, D, 0) == H * 2 * S * S * 4        # darkforest-cuda/src/lib.rs:2019-2027
    assert L.df_attn_workspace_bytes(3, 1, H, S, D, 0) == (S * H * D + 2 * H * S) * 4
    assert L.df_attn_workspace_bytes(4, 1, H, 1000, D, 256) == H * 4 * (2 + D) * 4
    assert L.df_attn_workspace_bytes(4, 1, H, 1000, D, 0) == 0 and L.df_attn_workspace_bytes(99, B, H, S, D, 0) == 0
    # no 32-bit overflow at the long-context sizes
    assert L.df_attn_workspace_bytes(2, 1, 12, 131072, 64, 0) == 12 * 2 * 131072 * 131072 * 4


def test_explicit_work_lists_cover_every_item_and_beat_the_round_robin_order():
    """df_attn_schedule_build (the MULTIFIT assignment the persistent kernels receive for mid-sized causal
    problems): every item exactly once, the heaviest CTA within 2 % of the average load where the round-robin
    order is 12 % off, and no table where it would not help."""
    import ctypes
    L = pkg().lib()

    def build(w, grid):
        arr = (ctypes.c_uint32 * len(w))(*w)
        off = (ctypes.c_uint16 * (grid + 1))()
        items = (ctypes.c_uint16 * len(w))()
        used = L.df_attn_schedule_build(ctypes.cast(arr, ctypes.c_void_p), len(w), grid, ctypes.cast(off, ctypes.c_void_p),
                                        ctypes.cast(items, ctypes.c_void_p))
        return used, list(off), list(items)

    # forward at S = 8192, B*H = 12: 32 pairs per head, weight 4 * key tiles + 3
    w = [4 * (2 * (31 - p) + 2) + 3 for p in range(32) for _ in range(12)]
    used, off, items = build(w, 148)
    assert used == 1 and off[0] == 0 and off[148] == len(w)
    assert sorted(items) == list(range(len(w)))
    loads = [sum(w[i] for i in items[off[c]:off[c + 1]]) for c in range(148)]
    avg = sum(w) / 148
    assert max(loads) <= 1.02 * avg, (max(loads), avg)
    snake = [0] * 148
    for k in range(len(w)):
        r, c = divmod(k, 148)
        snake[147 - c if r % 2 else c] += w[k]
    assert max(snake) >= 1.10 * avg                      # what the table is for
    for c in range(148):                                  # heaviest first within a CTA
        mine = [w[i] for i in items[off[c]:off[c + 1]]]
        assert mine == sorted(mine, reverse=True)
    assert build([5] * 100, 148)[0] == 0                  # one round at most: nothing to balance
    assert build([5] * 3000, 148)[0] == 0                 # too many items for the table
    # the step shape (S = 1024, B*H = 96): all loads are even numbers of steps, 14 is optimal either way
    w = [4 * (2 * (3 - p) + 2) + 3 for p in range(4) for _ in range(96)]
    used, off, items = build(w, 148)
    if used:
        assert sorted(items) == list(range(len(w)))


def test_options_and_simt_grid_limit_on_the_host():
    """Host-only behaviour of two entry points: df_attn_set_option returns the previous value and rejects unknown
    options; the SIMT launchers refuse batch * heads > 65535 (their grid's y dimension) with DF_ERR_UNSUPPORTED
    before any CUDA call is made (the pointers below are never dereferenced)."""
    import ctypes
    p = pkg()
    L = p.lib()
    prev = L.df_attn_set_option(p.OPT_FWD_PERSIST, 2)
    assert prev in (0, 1, 2)
    assert L.df_attn_get_option(p.OPT_FWD_PERSIST) == 2
    assert L.df_attn_set_option(p.OPT_FWD_PERSIST, prev) == 2
    assert L.df_attn_set_option(99, 1) == -1 and L.df_attn_get_option(-1) == -1
    buf = (ctypes.c_float * 64)()
    ptr = ctypes.cast(buf, ctypes.c_void_p)
    prev_variant = L.df_attn_set_variant(p.VARIANT_SIMT)
    try:
        L.df_attn_last_status()
        st = L.df_attn_forward(ptr, ptr, ptr, ptr, None, 70000, 1, 1, 4, 0.5, 1, None)
        assert st == p.DF_ERR_UNSUPPORTED
        assert L.df_attn_last_status() == p.DF_ERR_UNSUPPORTED
    finally:
        L.df_attn_set_variant(prev_variant)


def test_rust_bindings_match_the_headers():
    """dark-forest_b200/host/rust/kernels_attention.rs is the binding text for the reference's own host language. No
    Rust toolchain exists here, so its two extern "C" blocks are parsed as text and checked against the C headers:
    same symbols, same argument counts, and each argument's C type maps to the Rust type written there."""
    import os
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    rs = open(os.path.join(root, "dark-forest_b200", "host", "rust", "kernels_attention.rs")).read()
    ctype_to_rust = {"const float *": "*const f32", "float *": "*mut f32", "const void *": "*const c_void", "void *": "*mut c_void",
                     "const int32_t *": "*const i32", "const uint32_t *": "*const u32", "uint16_t *": "*mut u16",
                     "const char *": "*const c_char", "df_ring_t **": "*mut *mut DfRing", "const df_ring_t *": "*const DfRing",
                     "df_ring_t *": "*mut DfRing", "df_adamw_tensor_t *": "*mut DfAdamwTensor",
                     "const df_adamw_tensor_t *": "*const DfAdamwTensor", "int *": "*mut i32", "uint32_t": "u32", "int32_t": "i32", "int64_t": "i64",
                     "uint64_t": "u64", "long long": "i64", "float": "f32", "int": "i32", "void": None}

    def norm(ty):
        ty = " ".join(ty.replace("*", " * ").split())
        return re.sub(r"\* \*", "**", ty)

    rust = {}
    for body in re.findall(r'extern "C" \{(.*?)\n\}', rs, flags=re.S):
        for m in re.finditer(r"pub fn (\w+)\((.*?)\)\s*(?:->\s*([^;]+))?;", body, flags=re.S):
            args = [a.split(":", 1)[1].strip() for a in " ".join(m.group(2).split()).split(", ") if ":" in a]
            rust[m.group(1)] = (args, (m.group(3) or "").strip() or None)
    declared = {}
    for header in ("darkforest_kernels.h", "darkforest_ring.h"):
        text = re.sub(r"/\*.*?\*/", "", open(os.path.join(root, "include", header)).read(), flags=re.S)
        for m in re.finditer(r"DF_API\s+([\w\s\*]+?)\b(\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
            ret, name, args = norm(m.group(1)), m.group(2), " ".join(m.group(3).split())
            types = []
            for a in args.split(","):
                a = a.strip()
                if a in ("", "void"):
                    continue
                types.append(norm(re.match(r"(.*?)(\w+)$", a).group(1)))
            declared[name] = ([ctype_to_rust[t] for t in types], ctype_to_rust[ret])
    assert set(rust) == set(declared), set(rust) ^ set(declared)
    for name, (args, ret) in declared.items():
        assert rust[name] == (args, ret), (name, rust[name], (args, ret))
    # the wrappers call what they declare
    for wrapper in ("cuda_attn_forward_lse", "cuda_attn_backward_lse", "cuda_linear_qkv", "cuda_sync_checked"):
        assert f"pub fn {wrapper}(" in rs
