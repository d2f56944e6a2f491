"""On-disk format of a quantized checkpoint (include/vpq_safetensors.hpp): builds and runs the C++
test, then re-parses the directory it wrote with nothing but struct + json, as any other
safetensors reader would, and checks the layout rules of the reference's writer
(generative-models/quantize/safetensors-writer.cc:127-279)."""
import json
import os
import shutil
import struct
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "test_safetensors.cc")
OUT = os.path.join(ROOT, "tests", "cpp", "build", "test_safetensors")


def test_safetensors_writer_and_reader(tmp_path):
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    subprocess.run([shutil.which("g++") or "g++", "-std=c++17", "-O1", "-Wall", SRC, "-o", OUT,
                    f"-I{ROOT}/include"], check=True)
    r = subprocess.run([OUT, str(tmp_path)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "ALL PASSED" in r.stdout, r.stdout + r.stderr

    model = tmp_path / "model"
    index = json.loads((model / "model.safetensors.index.json").read_text())
    assert index["metadata"] == {"total_size": 0}
    shards = sorted(set(index["weight_map"].values()))
    assert len(shards) >= 2 and shards[0] == f"model-00001-of-{len(shards):05d}.safetensors"
    cfg = json.loads((model / "config.json").read_text())
    assert cfg["quantization"] == {"group_size": 64, "bits": 4}
    seen = {}
    for name in shards:
        raw = (model / name).read_bytes()
        (hlen,) = struct.unpack("<Q", raw[:8])
        assert (8 + hlen) % 16 == 0                     # the blob starts 16-byte aligned
        header = json.loads(raw[8:8 + hlen])            # trailing spaces are valid JSON whitespace
        blob = raw[8 + hlen:]
        ranges = sorted(tuple(v["data_offsets"]) for v in header.values())
        assert ranges[0][0] == 0 and ranges[-1][1] == len(blob)
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))   # no gaps, no overlap
        for k, v in header.items():
            assert index["weight_map"][k] == name
            n = 1
            for d in v["shape"]:
                n *= d
            width = {"U32": 4, "F32": 4, "F16": 2, "BF16": 2}[v["dtype"]]
            assert v["data_offsets"][1] - v["data_offsets"][0] == n * width
            seen[k] = v
    pfx = "model.layers.0.self_attn.q_proj"
    assert seen[pfx + ".weight"]["dtype"] == "U32" and seen[pfx + ".weight"]["shape"] == [48, 256 * 4 // 32]
    assert seen[pfx + ".scales"]["dtype"] == "F16" and seen[pfx + ".scales"]["shape"] == [48, 4]
    assert seen[pfx + ".biases"]["shape"] == [48, 4]
    assert seen["model.layers.0.mlp.down_proj.weight"]["shape"] == [16, 128 * 8 // 32]   # a w8 tensor beside w4 ones


def test_python_reader_reads_what_the_cpp_writer_wrote_and_back(tmp_path):
    """vpipe_b200.checkpoint (the Python twin) on the C++ writer's directory, then its own
    writer -> reader round trip byte for byte."""
    import numpy as np
    from vpipe_b200 import checkpoint
    if not os.path.exists(OUT):
        test_safetensors_writer_and_reader(tmp_path)
    else:
        subprocess.run([OUT, str(tmp_path)], check=True, capture_output=True)
    m = checkpoint.Model(str(tmp_path / "model"))
    assert m.quantization == {"group_size": 64, "bits": 4}
    assert m.quant_shape("model.layers.0.self_attn.q_proj") == (48, 256, 4, 64)
    assert m.quant_shape("model.layers.0.mlp.down_proj") == (16, 128, 8, 64)     # width from shapes alone
    assert m.numpy("model.norm.weight").tolist() == [1.0, 2.0, 3.0, 4.0, 5.0]

    rng = np.random.default_rng(5)
    tensors = {
        "a.weight": rng.integers(0, 2**32, (32, 16), dtype=np.uint32),
        "a.scales": rng.standard_normal((32, 2)).astype(np.float16),
        "a.biases": rng.standard_normal((32, 2)).astype(np.float16),
        "odd": np.arange(5, dtype=np.float32),
        "b.weight": rng.integers(0, 2**32, (64, 64), dtype=np.uint32),
    }
    out = tmp_path / "py"
    checkpoint.write_model(str(out), tensors, 64, 4, shard_max_bytes=4096)
    back = checkpoint.Model(str(out))
    for k, a in tensors.items():
        assert np.array_equal(np.asarray(back.numpy(k)), a), k
    assert back.quant_shape("a") == (32, 128, 4, 64)
