"""bitsandbytes-format NF4 weights in .safetensors files: container round trip and quant-state import (CPU)."""
from __future__ import annotations

import json
import struct

import pytest
import torch

from oracle import molt_oracle as oracle
from molt_b200.core.errors import CapabilityError
from molt_b200.methods.quant_state import NestedState, QuantState
from molt_b200.training import (bnb_nf4_weight, export_bnb_nf4_weight, nf4_weight_prefixes, read_safetensors,
                                write_safetensors)


def _quantised(n, k, nested, seed=5):
    gen = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=gen) * 0.02
    q = oracle.nf4_quantize(w, 64, oracle.HIGH_FIRST)
    if nested:
        nest = oracle.nest_absmax(q.scales)
        state = QuantState(absmax=nest.codes, shape=(n, k), nested=True,
                           state2=NestedState(nest.absmax2, nest.code2, nest.block2), offset=nest.offset)
        scales = oracle.resolve_nested_absmax(nest)
    else:
        state = QuantState(absmax=q.scales, shape=(n, k))
        scales = q.scales
    return q, state, scales


def test_container_round_trip_and_layout(tmp_path):
    tensors = {"a": torch.arange(12, dtype=torch.float32).reshape(3, 4), "b.c": torch.tensor([1, 2, 255], dtype=torch.uint8),
               "h": torch.randn(5, 2).bfloat16(), "e": torch.empty(0, 3, dtype=torch.int64), "s": torch.tensor(7, dtype=torch.int32)}
    path = tmp_path / "t.safetensors"
    write_safetensors(path, tensors, metadata={"format": "pt"})
    raw = path.read_bytes()
    (header_bytes,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + header_bytes])
    assert header_bytes % 8 == 0 and header["__metadata__"] == {"format": "pt"}
    assert header["a"] == {"dtype": "F32", "shape": [3, 4], "data_offsets": [0, 48]}
    assert header["h"]["dtype"] == "BF16" and header["s"]["shape"] == []
    back = read_safetensors(path)
    assert set(back) == set(tensors)
    for name, tensor in tensors.items():
        assert back[name].dtype == tensor.dtype and back[name].shape == tensor.shape and torch.equal(back[name], tensor)
    assert set(read_safetensors(path, names=["a"])) == {"a"}
    with pytest.raises(KeyError):
        read_safetensors(path, names=["nope"])


def test_container_rejects_damage(tmp_path):
    path = tmp_path / "bad.safetensors"
    path.write_bytes(b"\x01\x02")
    with pytest.raises(ValueError):
        read_safetensors(path)
    header = json.dumps({"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 8)     # 8 bytes where 16 are declared
    with pytest.raises(ValueError):
        read_safetensors(path)
    header = json.dumps({"x": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 4)
    with pytest.raises(CapabilityError):
        read_safetensors(path)


@pytest.mark.parametrize("nested", [False, True])
def test_bnb_layout_round_trip_dequantises_to_the_same_weight(tmp_path, nested):
    q, state, scales = _quantised(128, 192, nested)
    name = "model.layers.0.self_attn.q_proj.base_layer.weight"
    entries = export_bnb_nf4_weight(name, q.packed, state)
    assert name + ".quant_state.bitsandbytes__nf4" in entries and (name + ".nested_absmax" in entries) == nested
    entries["model.norm.weight"] = torch.ones(192).bfloat16()
    path = tmp_path / "model.safetensors"
    write_safetensors(path, entries)
    tensors = read_safetensors(path)
    assert nf4_weight_prefixes(tensors) == [name]
    packed, got = bnb_nf4_weight(tensors, name)
    assert packed.shape == (128 * 192 // 2, 1) and torch.equal(packed.reshape(-1), q.packed.reshape(-1))
    assert got.shape == (128, 192) and got.nested == nested and got.nibble_order == "high-first" and got.blocksize == 64
    assert torch.equal(got.code, state.code) and torch.equal(got.absmax, state.absmax)
    if nested:
        assert got.absmax.dtype == torch.uint8 and got.state2.blocksize == 256 and float(got.offset) == float(state.offset)
        nest = oracle.NestedAbsmax(got.absmax, got.state2.absmax, got.state2.code, float(got.offset), got.state2.blocksize)
        resolved = oracle.resolve_nested_absmax(nest)
    else:
        resolved = got.absmax
    assert torch.equal(resolved, scales)
    again = oracle.OracleNF4(packed.reshape(-1), resolved, (128, 192), 64, 128 * 192, oracle.HIGH_FIRST)
    assert torch.equal(oracle.nf4_dequantize(again), oracle.nf4_dequantize(q, torch.float32, scales))


def test_bnb_import_refuses_what_the_path_does_not_cover():
    q, state, _ = _quantised(64, 64, False)
    name = "w.weight"
    entries = export_bnb_nf4_weight(name, q.packed, state)

    def with_meta(**changes):
        meta = json.loads(bytes(entries[name + ".quant_state.bitsandbytes__nf4"].tolist()).decode())
        meta.update(changes)
        out = dict(entries)
        out[name + ".quant_state.bitsandbytes__nf4"] = torch.tensor(list(json.dumps(meta).encode()), dtype=torch.uint8)
        return out

    with pytest.raises(CapabilityError):
        bnb_nf4_weight(with_meta(quant_type="fp4"), name)
    with pytest.raises(CapabilityError):
        bnb_nf4_weight(with_meta(blocksize=128), name)
    with pytest.raises(ValueError):
        bnb_nf4_weight(with_meta(shape=[64, 64, 1]), name)
    with pytest.raises(ValueError):
        bnb_nf4_weight(with_meta(shape=[128, 64]), name)       # more elements than bytes and absmax cover
    missing = dict(entries)
    del missing[name + ".absmax"]
    with pytest.raises(KeyError):
        bnb_nf4_weight(missing, name)
    low_first = QuantState(absmax=state.absmax, shape=state.shape, nibble_order="low-first")
    with pytest.raises(CapabilityError):
        export_bnb_nf4_weight(name, q.packed, low_first)


def test_static_microbatch_runner_needs_cuda():
    """Without a GPU the captured micro-batch runner refuses to be built (reference training/static_cuda_graph.py:156-157)."""
    from molt_b200.training import StaticCudaMicrobatch, TensorSignature

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    p = torch.nn.Parameter(torch.ones(2))
    with pytest.raises(CapabilityError):
        StaticCudaMicrobatch(lambda x: (x * p).sum(), (torch.ones(2),), [p])
    sig = TensorSignature.of(torch.zeros(3, 4, dtype=torch.bfloat16))
    assert sig.shape == (3, 4) and sig.dtype == torch.bfloat16 and sig == TensorSignature((3, 4), torch.bfloat16, torch.device("cpu"))
