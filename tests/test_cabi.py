"""The C-ABI library loads and exports every symbol `include/mkb200.h` declares (no GPU needed)."""

import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "mkb200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mkb_[a-z_0-9]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("mkb_launch", "mkb_sync_status", "mkb_validate_instructions", "mkb_last_error",
                 "mkb_sm_count", "mkb_smem_bytes", "mkb_block_threads", "mkb_abi_version",
                 "mkb_launch_no_alloc", "mkb_sync_status_no_alloc", "mkb_peer_alloc", "mkb_peer_open", "mkb_peer_close", "mkb_peer_free"):
        assert must in names


def test_library_exports_every_declared_symbol():
    import __graft_entry__ as entry

    entry.build()
    lib = ctypes.CDLL(str(ROOT / "megakernels_b200" / "native" / "libmkb200.so"))
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in mkb200.h but not exported"
    lib.mkb_abi_version.restype = ctypes.c_int
    assert lib.mkb_abi_version() == 4
    lib.mkb_smem_bytes.restype = ctypes.c_int
    assert 0 < lib.mkb_smem_bytes() <= 227 * 1024


def test_struct_layout_matches_between_header_and_shim():
    """Field names and order of MkbGlobals in the ctypes shim equal the header's."""
    import sys

    sys.path.insert(0, str(ROOT / "megakernels_b200" / "native"))
    import mk_llama

    text = (ROOT / "include" / "mkb200.h").read_text()
    body = text[text.index("typedef struct MkbGlobals {") : text.index("} MkbGlobals;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = re.findall(r"[\w\*]\s+\**(\w+)(?:\[\w+\])?;", body)
    assert names == [f[0] for f in mk_llama.MkbGlobals._fields_]
    body = text[text.index("typedef struct MkbTensorParallel {") : text.index("} MkbTensorParallel;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = re.findall(r"[\w\*]\s+\**(\w+)(?:\[\w+\])?;", body)
    assert names == [f[0] for f in mk_llama.MkbTensorParallel._fields_]
    # size agreed with the compiled library: validate() compares struct_bytes with sizeof
    assert ctypes.sizeof(mk_llama.MkbTensorParallel) == 16 + 2 * 8 * 8 + 16


def test_host_validation_without_a_gpu():
    """mkb_validate_instructions is pure host code: it must reject a bad schedule here."""
    import sys

    import torch

    sys.path.insert(0, str(ROOT / "megakernels_b200" / "native"))
    import mk_llama

    lib = mk_llama.load_library()
    g = mk_llama.MkbGlobals()
    g.abi_version = 0
    lib.mkb_validate_instructions.argtypes = [ctypes.POINTER(mk_llama.MkbGlobals), ctypes.c_void_p]
    lib.mkb_validate_instructions.restype = ctypes.c_int
    buf = torch.zeros(1, 1, 32, dtype=torch.int32)
    rc = lib.mkb_validate_instructions(ctypes.byref(g), ctypes.c_void_p(buf.data_ptr()))
    assert rc == 1 and b"ABI version" in lib.mkb_last_error()
    # with the right version the library compares struct sizes next: the ctypes layout must
    # have the size the compiler gave the header's struct, so the complaint moves on to pointers
    g.abi_version = mk_llama.MKB_ABI_VERSION
    g.struct_bytes = ctypes.sizeof(mk_llama.MkbGlobals)
    rc = lib.mkb_validate_instructions(ctypes.byref(g), ctypes.c_void_p(buf.data_ptr()))
    assert rc == 1 and b"barriers is NULL" in lib.mkb_last_error()


def test_host_validation_of_all_reduce_instructions():
    """Opcode 8 is only legal with the tensor-parallel block filled in, and its chunk index
    must stay below tp.num_chunks (pure host code: fake, aligned, non-NULL pointers suffice)."""
    import sys

    import torch

    sys.path.insert(0, str(ROOT / "megakernels_b200" / "native"))
    import mk_llama

    lib = mk_llama.load_library()
    lib.mkb_validate_instructions.argtypes = [ctypes.POINTER(mk_llama.MkbGlobals), ctypes.c_void_p]
    lib.mkb_validate_instructions.restype = ctypes.c_int
    g = mk_llama.MkbGlobals()
    g.abi_version = mk_llama.MKB_ABI_VERSION
    g.struct_bytes = ctypes.sizeof(mk_llama.MkbGlobals)
    fake = 0x10000
    for name, ctype in mk_llama.MkbGlobals._fields_:
        if ctype is ctypes.c_void_p and name not in ("timings", "status", "pos_id_device", "argmax_out"):
            setattr(g, name, fake)
    g.num_sms, g.queue_len, g.barrier_ops, g.barrier_width = 1, 2, 10, 48
    g.num_layers, g.hidden_size, g.intermediate_size, g.head_dim = 2, 2048, 8192, 64
    g.num_attention_heads, g.num_kv_heads, g.vocab_size = 32, 8, 128256
    g.kv_max_len, g.kv_batch, g.max_partials, g.matvec_reduction_size = 128, 1, 4, 2048
    ins = torch.zeros(1, 2, 32, dtype=torch.int32)
    ins[0, 0, :5] = torch.tensor([8, 1, 0, 3, 4])

    def check():
        rc = lib.mkb_validate_instructions(ctypes.byref(g), ctypes.c_void_p(ins.data_ptr()))
        return rc, lib.mkb_last_error().decode()

    rc, msg = check()
    assert rc == 1 and "without tensor parallelism" in msg
    g.tp.size, g.tp.rank, g.tp.num_chunks = 2, 1, 4
    for r in range(2):
        g.tp.hidden_ll_peers[r] = fake
        g.tp.recv_peers[r] = fake
    g.tp.partial = fake
    rc, msg = check()
    assert rc == 1 and "epoch_device" in msg
    g.tp.epoch_device = fake
    assert check()[0] == 0
    ins[0, 0, 3] = 4  # chunk == num_chunks
    rc, msg = check()
    assert rc == 1 and "chunk outside" in msg
    ins[0, 0, 3] = 0
    g.tp.num_chunks = 3  # not a multiple of the group size
    rc, msg = check()
    assert rc == 1 and "num_chunks" in msg


def test_host_validation_of_attention_reduction_modes():
    """skip_attn_reduction: 0 / 1 / 2 are the only values; mode 2 (the last partial merges) has no
    AttentionReduction instructions; mode 1 has exactly one partition (pure host code)."""
    import sys

    import torch

    sys.path.insert(0, str(ROOT / "megakernels_b200" / "native"))
    import mk_llama

    lib = mk_llama.load_library()
    lib.mkb_validate_instructions.argtypes = [ctypes.POINTER(mk_llama.MkbGlobals), ctypes.c_void_p]
    lib.mkb_validate_instructions.restype = ctypes.c_int
    g = mk_llama.MkbGlobals()
    g.abi_version = mk_llama.MKB_ABI_VERSION
    g.struct_bytes = ctypes.sizeof(mk_llama.MkbGlobals)
    fake = 0x10000
    for name, ctype in mk_llama.MkbGlobals._fields_:
        if ctype is ctypes.c_void_p and name not in ("timings", "status", "pos_id_device", "argmax_out"):
            setattr(g, name, fake)
    g.num_sms, g.queue_len, g.barrier_ops, g.barrier_width = 1, 2, 10, 48
    g.num_layers, g.hidden_size, g.intermediate_size, g.head_dim = 2, 2048, 8192, 64
    g.num_attention_heads, g.num_kv_heads, g.vocab_size = 32, 8, 128256
    g.kv_max_len, g.kv_batch, g.max_partials, g.matvec_reduction_size = 128, 1, 4, 2048
    ins = torch.zeros(1, 2, 32, dtype=torch.int32)
    ins[0, 0, :6] = torch.tensor([2, 0, 1, 3, 2, 0])  # partial 2 of 3, KV head 1
    ins[0, 1, :9] = torch.tensor([3, 0, 4, 3, 1, 3, 0, 1, 2])  # terminal reduction of heads 4..7

    def check(mode):
        g.skip_attn_reduction = mode
        rc = lib.mkb_validate_instructions(ctypes.byref(g), ctypes.c_void_p(ins.data_ptr()))
        return rc, lib.mkb_last_error().decode()

    assert check(0)[0] == 0
    rc, msg = check(1)
    assert rc == 1 and "num_partials == 1" in msg
    rc, msg = check(2)
    assert rc == 1 and "AttentionReduction instruction" in msg
    rc, msg = check(3)
    assert rc == 1 and "0, 1 or 2" in msg
    ins[0, 1].zero_()  # without the reduction instruction mode 2 is a valid stream
    assert check(2)[0] == 0
