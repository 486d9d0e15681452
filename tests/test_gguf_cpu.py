"""GGUF container and block codecs on CPU: round trips, block geometry, agreement with the `gguf` Python package
(ggml's reference dequantisers) when it is importable, and the checkpoint round trip of a whole model."""
import struct

import numpy as np
import pytest
import torch

from llaminar_b200.gguf import GGMLType, GGUFFile, GGUFWriter, dequantize, quantize
from llaminar_b200.gguf.constants import BLOCK_GEOMETRY
from llaminar_b200.gguf.reader import GGUFError

QUANT_TYPES = ["Q8_0", "Q4_0", "Q4_K", "Q5_K", "Q6_K", "IQ3_S"]
DEQUANT_ONLY = ["Q4_1", "Q5_0", "Q5_1", "IQ4_NL", "Q2_K", "Q3_K", "IQ4_XS", "IQ3_XXS", "IQ2_XXS", "IQ2_XS", "IQ2_S", "IQ1_S", "IQ1_M"]
EXPECTED_BLOCKS = {"Q8_0": (32, 34), "Q4_0": (32, 18), "Q4_1": (32, 20), "Q5_0": (32, 22), "Q5_1": (32, 24), "IQ4_NL": (32, 18),
                   "Q4_K": (256, 144), "Q5_K": (256, 176), "Q6_K": (256, 210), "Q3_K": (256, 110), "Q2_K": (256, 84),
                   "IQ4_XS": (256, 136), "IQ3_S": (256, 110), "IQ3_XXS": (256, 98), "IQ2_XXS": (256, 66), "IQ2_XS": (256, 74),
                   "IQ2_S": (256, 82), "IQ1_S": (256, 50), "IQ1_M": (256, 56)}


def test_block_geometry_matches_ggml():
    for name, geo in EXPECTED_BLOCKS.items():
        assert BLOCK_GEOMETRY[GGMLType[name]] == geo, name


@pytest.mark.parametrize("name", QUANT_TYPES)
def test_quantize_dequantize_error_is_bounded(name):
    qt = GGMLType[name]
    g = torch.Generator().manual_seed(1)
    x = torch.randn(8, 512, generator=g) * 0.02
    raw = quantize(x, qt)
    e, b = BLOCK_GEOMETRY[qt]
    assert raw.numel() == x.numel() // e * b and raw.dtype == torch.uint8
    y = dequantize(raw, qt, tuple(x.shape))
    rel = ((y - x).norm() / x.norm()).item()
    assert rel < {"Q8_0": 0.01, "Q6_K": 0.02, "Q5_K": 0.04, "Q4_K": 0.08, "Q4_0": 0.12, "IQ3_S": 0.2}[name]
    assert torch.equal(quantize(y, qt), quantize(y, qt))           # deterministic


@pytest.mark.parametrize("name", QUANT_TYPES + DEQUANT_ONLY)
def test_dequantize_agrees_with_ggml_reference(name):
    gq = pytest.importorskip("gguf.quants")
    import gguf
    qt = GGMLType[name]
    gt = getattr(gguf.GGMLQuantizationType, name)
    e, b = BLOCK_GEOMETRY[qt]
    rng = np.random.default_rng(3)
    raw = rng.integers(0, 256, size=(4, 512 // e * b), dtype=np.uint8)
    # keep every fp16 scale field finite: clear the top exponent bit of all 16-bit words
    raw16 = raw.view(np.uint16)
    raw16 &= 0x3FFF
    try:
        ref = gq.dequantize(raw, gt)
    except (NotImplementedError, KeyError):
        pytest.skip(f"the gguf package has no reference dequantiser for {name}")
    ours = dequantize(torch.from_numpy(raw.reshape(-1).copy()), qt, (4, 512)).numpy()
    np.testing.assert_allclose(ours, ref.reshape(4, 512), rtol=1e-6, atol=1e-7)


def test_container_round_trip_and_value_types(tmp_path):
    w = GGUFWriter()
    w.add("general.architecture", "qwen3")
    w.add("qwen3.block_count", 2)
    w.add("qwen3.rope.freq_base", 1e6)
    w.add("flag", True)
    w.add("tokenizer.ggml.tokens", ["a", "b", "çé"])
    w.add("ints", [1, 2, 3])
    x = torch.arange(2 * 256, dtype=torch.float32).view(2, 256) / 100
    w.add_tensor("blk.0.attn_q.weight", x, GGMLType.Q8_0)
    w.add_tensor("output_norm.weight", torch.ones(256), GGMLType.F32)
    path = tmp_path / "m.gguf"
    w.write(str(path))
    data = path.read_bytes()
    assert data[:4] == b"GGUF" and struct.unpack("<I", data[4:8])[0] == 3
    f = GGUFFile(str(path))
    assert f.architecture == "qwen3" and f.get("qwen3.block_count") == 2 and f.get("flag") is True
    assert f.get("tokenizer.ggml.tokens") == ["a", "b", "çé"] and f.get("ints") == [1, 2, 3]
    t = f["blk.0.attn_q.weight"]
    assert tuple(t.shape) == (2, 256) and t.qtype == GGMLType.Q8_0           # dims are stored reversed on disk
    assert torch.allclose(t.to_float(), x, atol=0.03)
    assert (t.offset % 32) == 0                                               # data section alignment
    f.close()


def test_reader_rejects_bad_files(tmp_path):
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"NOPE" + b"\0" * 64)
    with pytest.raises(GGUFError):
        GGUFFile(str(p))
    p.write_bytes(b"GGUF" + struct.pack("<I", 99) + b"\0" * 64)
    with pytest.raises(GGUFError):
        GGUFFile(str(p))


def test_model_checkpoint_round_trip(tmp_path):
    from llaminar_b200.models.config import SHAPES
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.models.weights import ModelWeights
    w = synthesize(SHAPES["tiny-qwen3moe"], "Q4_K_M", seed=3)
    path = tmp_path / "tiny.gguf"
    w.save_gguf(str(path))
    r = ModelWeights.from_gguf(str(path))
    assert r.config.n_experts == w.config.n_experts and r.config.d_model == w.config.d_model
    for name in ("blk.0.ffn_gate_exps.weight", "blk.1.attn_q.weight", "token_embd.weight"):
        assert r[name].qtype == w[name].qtype and torch.equal(r[name].raw.cpu(), w[name].raw.cpu())
    assert "tokenizer.ggml.tokens" in r.metadata



def test_checkpoint_with_two_bit_and_one_bit_tensors_loads_and_runs(tmp_path):
    """A file whose projections use the 2-bit / 1-bit codebook formats (no quantiser here: random valid blocks) goes
    through the loader and the engine; the tokens are those of the fp32 oracle on the same decoded weights."""
    from llaminar_b200.engine.engine import LLMEngine
    from llaminar_b200.engine.sampling import SamplingParams
    from llaminar_b200.models.config import SHAPES
    from llaminar_b200.models.reference import ReferenceModel
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.models.weights import ModelWeights, QTensor
    w = synthesize(SHAPES["tiny-qwen3"], "Q8_0", seed=1)
    rng = np.random.default_rng(5)
    swaps = {"blk.0.ffn_gate.weight": "IQ2_XXS", "blk.0.ffn_up.weight": "IQ2_XS", "blk.0.ffn_down.weight": "IQ2_S",
             "blk.1.ffn_gate.weight": "IQ1_S", "blk.1.ffn_up.weight": "IQ1_M"}
    for name, fmt in swaps.items():
        qt = GGMLType[fmt]
        n, k = w[name].shape
        assert k % 256 == 0
        e, b = BLOCK_GEOMETRY[qt]
        raw = rng.integers(0, 256, size=(n * k // e, b), dtype=np.uint8)
        raw16 = raw.view(np.uint16) if b % 2 == 0 else None
        # small finite super-block scales: overwrite the fp16 field (IQ1_M spreads it over the scale words' top nibbles)
        d = np.float16(0.002).view(np.uint16)
        if fmt == "IQ1_M":
            sc = raw[:, 48:56].copy().view(np.uint16)
            for i in range(4):
                sc[:, i] = (sc[:, i] & 0x0FFF) | (((d >> (4 * i)) & 0xF) << 12)
            raw[:, 48:56] = sc.view(np.uint8)
        else:
            raw[:, 0:2] = np.array([d], dtype=np.uint16).view(np.uint8)
        w.tensors[name] = QTensor(qt, (n, k), torch.from_numpy(raw.reshape(-1).copy()))
    path = str(tmp_path / "lowbit.gguf")
    w.save_gguf(path)
    r = ModelWeights.from_gguf(path)
    for name, fmt in swaps.items():
        assert r[name].qtype == GGMLType[fmt]
        t = r[name].to_float()
        assert torch.isfinite(t).all() and 0 < t.abs().max() < 1.0
    eng = LLMEngine.from_gguf(path, device="cpu", max_batch=1, max_context=128)
    prompt = list(range(3, 35))
    out = eng.generate([prompt], SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))[0]
    assert out == ReferenceModel(r).generate_greedy(torch.tensor(prompt), 8)[0]


def test_expert_stacks_without_a_packed_layout_are_reencoded_for_the_grouped_kernels():
    from llaminar_b200.engine.cuda_model import expert_tensors_for_packing
    from llaminar_b200.models.config import SHAPES
    from llaminar_b200.models.synth import synthesize
    from llaminar_b200.models.weights import QTensor
    from llaminar_b200.ops.layout import can_pack
    w = synthesize(SHAPES["tiny-qwen3moe"], "Q4_K_M", seed=2)
    p = "blk.0."
    before = [w[p + n] for n in ("ffn_gate_exps.weight", "ffn_up_exps.weight", "ffn_down_exps.weight")]
    if before[0].qtype == before[1].qtype:
        got = expert_tensors_for_packing(w, p)
        assert all(a is b for a, b in zip(got, before))                  # packable formats pass through untouched
    # a 2-bit gate stack: gate and up move to Q8_0 together, down stays as it is
    E, ff, d = before[0].shape
    rng = np.random.default_rng(7)
    raw = rng.integers(0, 256, size=(E * ff * d // 256, 74), dtype=np.uint8)
    raw[:, 0:2] = np.array([np.float16(0.003)], dtype=np.float16).view(np.uint8)
    low = QTensor(GGMLType.IQ2_XS, (E, ff, d), torch.from_numpy(raw.reshape(-1).copy()))
    w.tensors[p + "ffn_gate_exps.weight"] = low
    ge, ue, de = expert_tensors_for_packing(w, p)
    assert ge.qtype == ue.qtype == GGMLType.Q8_0 and can_pack(ge.qtype, d) and de is before[2]
    assert w[p + "ffn_gate_exps.weight"] is ge                            # cached for the other expert-parallel slabs
    a, b = low.to_float(), ge.to_float()
    assert a.shape == b.shape and ((a - b).norm() / a.norm()).item() < 0.01
    u0, u1 = before[1].to_float(), ue.to_float()
    assert ((u0 - u1).norm() / u0.norm()).item() < 0.01


def test_block_formats_without_a_packed_layout_are_reencoded_for_the_dense_kernels():
    from llaminar_b200.engine.cuda_model import QLinear, for_kernels
    from llaminar_b200.models.weights import QTensor, qtensor_from_float
    from llaminar_b200.ops.layout import PackedWeight
    g = torch.Generator().manual_seed(0)
    x = torch.randn(128, 512, generator=g) * 0.02
    packed = qtensor_from_float(x, GGMLType.Q4_K)
    assert for_kernels(packed) is packed                                    # has a device layout: untouched
    half = qtensor_from_float(x, GGMLType.F16)
    assert for_kernels(half) is half                                        # unquantised: stays dense
    rng = np.random.default_rng(1)
    raw = rng.integers(0, 256, size=(128 * 512 // 256, 84), dtype=np.uint8)          # Q2_K: d and dmin are the last two fp16
    raw[:, 80:84] = np.array([np.float16(0.01), np.float16(0.005)], dtype=np.float16).view(np.uint8)
    low = QTensor(GGMLType.Q2_K, (128, 512), torch.from_numpy(raw.reshape(-1).copy()))
    t = for_kernels(low)
    assert t.qtype == GGMLType.Q8_0 and t.shape == (128, 512)
    a, b = low.to_float(), t.to_float()
    assert ((a - b).norm() / a.norm()).item() < 0.01
    narrow = QTensor(GGMLType.Q5_0, (64, 128), quantize(torch.randn(64, 128, generator=g), GGMLType.Q8_0)[:64 * 128 // 32 * 22])
    assert for_kernels(narrow) is narrow                                    # K is not a whole 256-column chunk: dense path
    lin = QLinear.from_qtensors([packed, low], "cpu")
    assert len(lin.parts) == 2 and all(isinstance(p, PackedWeight) for p, _ in lin.parts) and lin.n_out == 256


def test_files_written_here_are_read_by_the_gguf_package_and_its_files_by_us(tmp_path):
    """Interoperability of the container format in both directions: a checkpoint written by this package is opened with the
    `gguf` package's reader (metadata values, tensor names, shapes, types, bytes), and a file written with the `gguf`
    package's writer is opened with the reader here."""
    gguf = pytest.importorskip("gguf")
    import numpy as np
    from llaminar_b200.gguf import GGUFFile
    from llaminar_b200.models.config import SHAPES
    from llaminar_b200.models.synth import synthesize
    w = synthesize(SHAPES["tiny-qwen35"], "Q4_K_M", seed=1)
    path = str(tmp_path / "ours.gguf")
    w.save_gguf(path)
    r = gguf.GGUFReader(path)
    field = lambda k: r.fields[k]
    assert bytes(field("general.architecture").parts[-1]).decode() == "qwen35"
    assert int(field("qwen35.ssm.state_size").parts[-1][0]) == 32 and int(field("qwen35.full_attention_interval").parts[-1][0]) == 4
    assert len(field("tokenizer.ggml.tokens").data) == 1024
    names = {t.name: t for t in r.tensors}
    assert set(names) == set(w.tensors)
    for name in ("blk.0.attn_qkv.weight", "blk.3.attn_q.weight", "blk.0.ssm_a", "blk.0.ssm_conv1d.weight", "token_embd.weight"):
        t, ours = names[name], w[name]
        assert t.tensor_type.name == ours.qtype.name
        assert list(reversed([int(x) for x in t.shape])) == list(ours.shape)            # GGUF lists the fastest dimension first
        assert np.array_equal(np.asarray(t.data).reshape(-1).view(np.uint8), ours.raw.numpy())
    # the other direction
    theirs = str(tmp_path / "theirs.gguf")
    wr = gguf.GGUFWriter(theirs, "qwen3")
    wr.add_uint32("qwen3.block_count", 2)
    wr.add_float32("qwen3.rope.freq_base", 1e6)
    wr.add_array("tokenizer.ggml.tokens", ["a", "b", "c"])
    x = np.arange(24, dtype=np.float32).reshape(4, 6)
    wr.add_tensor("blk.0.ffn_norm.weight", x)
    wr.write_header_to_file()
    wr.write_kv_data_to_file()
    wr.write_tensors_to_file()
    wr.close()
    gf = GGUFFile(theirs)
    assert gf.architecture == "qwen3" and gf.get("qwen3.block_count") == 2 and gf.get("tokenizer.ggml.tokens") == ["a", "b", "c"]
    t = gf["blk.0.ffn_norm.weight"]
    assert tuple(t.shape) == (4, 6) and torch.equal(torch.frombuffer(bytearray(t.raw().numpy().tobytes()), dtype=torch.float32).view(4, 6), torch.from_numpy(x))
    gf.close()
