"""q3_decode_noalloc: the decode step for callers that cannot allocate device memory.

Some users of the library run where cudaMalloc is off limits (inside another runtime's memory budget,
or with all device memory carved up in advance), so they cannot create an engine.  This test calls
the allocation-free entry point through the C ABI, twice in a row, and checks each result against the
engine's q3_decode on the same inputs.  It is collected last on purpose."""
from __future__ import annotations

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_noalloc_matches_engine_twice_in_a_row(oracle):
    from qwen3mk import Megakernel, _cabi
    from qwen3mk.kernel import SeqTable, rope_rows

    lib = _cabi.load()
    shp = oracle.Shape(layers=2, vocab=2048)
    inp = oracle.synthetic(41, shp, context=50)
    dev = {k: v.cuda() for k, v in inp.items()}
    mk = Megakernel(layers=2, vocab=2048, path="layered", max_batch=2)
    rope = rope_rows(256, "cuda")
    w = _cabi.Weights(*[dev[n].data_ptr() for n in _cabi.WEIGHT_FIELDS])
    g = torch.Generator().manual_seed(3)
    for call in range(2):
        lens = [50, 17 + call]
        toks = torch.randint(0, 2048, (2,), generator=g).cuda()
        kcs = [dev["kcache"], dev["kcache"][:, :lens[1]].contiguous()]
        vcs = [dev["vcache"], dev["vcache"][:, :lens[1]].contiguous()]
        seqs = SeqTable(kcs, vcs)
        want = mk.bind_sequences(dev, toks, seqs)
        mk.launch()
        mk.status()
        logits = torch.full((2, 2048), float("nan"), device="cuda")
        nxt = torch.full((2,), -1, dtype=torch.int64, device="cuda")
        kw = torch.zeros((2, 2, 8, 128), dtype=torch.bfloat16, device="cuda")
        vw = torch.zeros_like(kw)
        a = _cabi.DecodeArgs(2, max(lens), _cabi.F_PATH_LAYERED, 0, toks.data_ptr(), seqs.seq_k.data_ptr(), seqs.seq_v.data_ptr(),
                             seqs.stride.data_ptr(), seqs.len.data_ptr(), logits.data_ptr(), nxt.data_ptr(), kw.data_ptr(), vw.data_ptr())
        rc = lib.q3_decode_noalloc(ctypes.byref(w), rope.data_ptr(), rope.shape[0], 2, 2048, ctypes.byref(a),
                                   torch.cuda.current_stream().cuda_stream)
        assert rc == 0, lib.q3_last_error(None)
        torch.cuda.synchronize()
        assert nxt.tolist() == want["next_token"].tolist()
        # same kernels, same order of operations: the tolerance of the parity tests is far more than needed
        assert oracle.rel_l2(logits, want["logits"]) <= 1e-4
        assert oracle.bf16_ulps(kw, want["k_write"]) <= 2 and oracle.bf16_ulps(vw, want["v_write"]) <= 2
        # and against the CPU oracle, like every other path
        refs = oracle.decode_batch(oracle.to_fp32(inp), toks.tolist(), [k.cpu() for k in kcs], [v.cpu() for v in vcs])
        for b, ref in enumerate(refs):
            assert int(nxt[b]) == int(ref["next_token"])
            assert oracle.rel_l2(logits[b], ref["logits"]) <= 1e-4

        words = (ctypes.c_uint32 * 8)()
        assert lib.q3_noalloc_status(torch.cuda.current_stream().cuda_stream, words, 8) == 0 and words[0] == 0

    # a token outside the vocabulary is replaced by token 0 and reported through the status call
    bad = torch.tensor([5, 10 ** 7], dtype=torch.int64, device="cuda")
    a.token = bad.data_ptr()
    assert lib.q3_decode_noalloc(ctypes.byref(w), rope.data_ptr(), rope.shape[0], 2, 2048, ctypes.byref(a),
                                 torch.cuda.current_stream().cuda_stream) == 0
    words = (ctypes.c_uint32 * 8)()
    assert lib.q3_noalloc_status(torch.cuda.current_stream().cuda_stream, words, 8) == _cabi.ERR_DEVICE_WAIT
    assert words[0] == 3 and b"code 3" in lib.q3_last_error(None)

    # sizes beyond the static scratch are refused, with a message
    a3 = _cabi.DecodeArgs(3, 10, _cabi.F_PATH_LAYERED, 0, 1, 1, 1, 1, 1, None, 1, None, None)
    assert lib.q3_decode_noalloc(ctypes.byref(w), rope.data_ptr(), rope.shape[0], 2, 2048, ctypes.byref(a3), None) == _cabi.ERR_INVALID
    assert b"at most 2" in lib.q3_last_error(None)
