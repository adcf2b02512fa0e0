"""A model loaded from a GGUF file (yuuka_model_load_gguf) against the same tensors handed over one
by one: identical logits, for the dense and the MoE layout (rank-3 expert tensors, [kernel, channels]
conv weights)."""
import numpy as np
import pytest

from yuuka_b200 import cuda, gguf_writer as gw, synth

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind", ["dense", "moe"])
def test_gguf_model_matches_tensor_by_tensor_model(tmp_path, kind):
    cfg = synth.tiny_config() if kind == "dense" else synth.tiny_moe_config()
    tensors = synth.make_model(cfg, "q8_0", seed=5, unit_norms=False)
    path = tmp_path / "model.gguf"
    gw.write(str(path), gw.config_metadata(cfg, tokens=(kind == "moe")), tensors, cfg=cfg)
    dev = cuda.Device(0)
    a = cuda.Model(dev, cfg, tensors)
    b = cuda.Model.from_gguf(dev, str(path))
    assert b.cfg["vocab"] == cfg["vocab"] and b.weight_bytes == a.weight_bytes
    prompt = synth.uniform_i32(9, 0, cfg["vocab"], 3).tolist()
    out = []
    for m in (a, b):
        sess = cuda.Session(m, max_batch=1, max_nodes=9, capacity=64, kv_format=cuda.KV_F32)
        out.append(sess.prefill_logits(prompt))
        sess.close()
    assert np.array_equal(out[0], out[1])
    a.close(); b.close()
    # a file that lacks a required tensor is refused with the tensor's name
    short = dict(tensors)
    del short["output_norm.weight"]
    gw.write(str(path), gw.config_metadata(cfg), short, cfg=cfg)
    with pytest.raises(cuda.YuukaError) as e:
        cuda.Model.from_gguf(dev, str(path))
    assert "output_norm.weight" in str(e.value)
    dev.close()
