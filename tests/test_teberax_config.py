"""CPU: the Teberax configuration, checkpoint names and shapes, the size that only a tensor's shape gives, and the row
permutation that lets two attention maps run as ordinary grouped heads - against ``oracle/teberax.py``."""
import json
import struct

import pytest
import torch

from oracle import teberax as O


def test_configuration_round_trip_shapes_and_names():
    from nano_qwen3tts_vllm_b200.config import TeberaxConfig
    from nano_qwen3tts_vllm_b200.models.registry import resolve
    from nano_qwen3tts_vllm_b200.models.teberax import TeberaxForCausalLM, checkpoint_shapes, random_state_dict
    cfg = O.random_config(types=("attention", "parallel", "latent_attention", "attention", "attention"), kv_from={3: 0, 4: 0},
                          ff=("moe", "dense", None, "moe", "dense"))
    assert resolve(cfg).name == "Teberax"
    c = TeberaxConfig.from_dict(cfg)
    assert c.to_dict() == cfg
    assert {k: tuple(v) for k, v in checkpoint_shapes(c).items()} == O.tensor_shapes(cfg)
    with torch.device("meta"):
        model = TeberaxForCausalLM(c)
    assert sorted(model.checkpoint_names()) == sorted(O.tensor_shapes(cfg))
    sd = random_state_dict(c, 3)
    assert {k: tuple(v.shape) for k, v in sd.items()} == O.tensor_shapes(cfg)
    plan = model.cache_plan()
    assert plan[3]["paged"] == [] and plan[4]["paged"] == [] and len(plan[0]["paged"]) == 2        # borrowed keys and values
    assert plan[1]["state"] and plan[2]["state"] == [] and len(plan[2]["paged"]) == 1


@pytest.mark.parametrize("bad", [
    lambda c: c["layers"][0].update(type="other"),
    lambda c: c["layers"][2]["mixer"].update(kv_from=3),                 # a later layer
    lambda c: c["layers"][2]["mixer"].update(kv_from=1),                 # not an attention layer
    lambda c: c["layers"][3]["mixer"].update(kv_from=2, vdim=4),         # other key/value sizes
    lambda c: c["layers"][2]["mixer"].update(heads=3),                   # 3 heads over 2 key/value heads
    lambda c: c["layers"][1]["mlp"]["router"].update(top=9),             # more choices than router outputs
    lambda c: c["layers"][1]["mixer"]["rot"].update(dims=6),             # more rotated coordinates than the rotated part
])
def test_configuration_errors(bad):
    from nano_qwen3tts_vllm_b200.config import TeberaxConfig
    cfg = json.loads(json.dumps(O.random_config()))
    bad(cfg)
    with pytest.raises(ValueError):
        TeberaxConfig.from_dict(cfg)


def test_absent_keys_mean_absent_mechanisms():
    from nano_qwen3tts_vllm_b200.config import TeberaxConfig
    cfg = json.loads(json.dumps(O.random_config()))
    del cfg["logit_softcap"], cfg["layers"][2]["mixer"]["mask"], cfg["layers"][1]["mixer"]["mask"]
    del cfg["layers"][0]["mixer"]["left"]["softcap"], cfg["layers"][0]["mixer"]["left"]["rot"]["scaling"]
    del cfg["layers"][3]["mixer"]["mask"]["keep_first"], cfg["layers"][1]["mlp"]["router"]["identity"]
    c = TeberaxConfig.from_dict(cfg)
    assert c.logit_softcap == 0 and c.layers[2].mixer.window == 0 and c.layers[2].mixer.keep_first == 0 and c.layers[1].mixer.window == 0
    left = c.layers[0].mixer.left
    assert left.softcap == 0 and left.rot.scaling is None and left.sink == "zero" and left.mask_size == 0
    assert c.layers[3].mixer.window == 9 and c.layers[3].mixer.keep_first == 0 and c.layers[1].mlp.identity == 0


def test_inner_size_of_the_decay_projection_comes_from_the_tensor_shape(tmp_path):
    from nano_qwen3tts_vllm_b200.config import load_model_config
    cfg = json.loads(json.dumps(O.random_config(right=dict(decay_rank=7))))
    del cfg["layers"][0]["mixer"]["right"]["decay_rank"]
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    header = json.dumps({"l0.mix.right.a1": {"dtype": "BF16", "shape": [7, cfg["width"]], "data_offsets": [0, 7 * cfg["width"] * 2]}}).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(header)) + header + bytes(7 * cfg["width"] * 2))
    assert load_model_config(str(tmp_path)).layers[0].mixer.right.decay_rank == 7


def test_map_major_rows_make_the_two_maps_ordinary_grouped_heads():
    """Head h's map m of the stored projection is query head m * H + h of the permuted one, and its key head
    (m * H + h) // (H / G) = m * G + h // (H / G) is map m of key/value head h // (H / G)."""
    from nano_qwen3tts_vllm_b200.layers.attention import DifferentialAttention
    H, G, d, D, T = 6, 2, 4, 10, 5
    g = torch.Generator().manual_seed(0)
    wq, wk, x = torch.randn(H * 2 * d, D, generator=g), torch.randn(G * 2 * d, D, generator=g), torch.randn(T, D, generator=g)
    q, k = (x @ wq.T).view(T, H, 2, d), (x @ wk.T).view(T, G, 2, d)
    q2 = (x @ DifferentialAttention.map_major(wq, H, d).T).view(T, 2 * H, d)
    k2 = (x @ DifferentialAttention.map_major(wk, G, d).T).view(T, 2 * G, d)
    for m in range(2):
        for h in range(H):
            assert torch.equal(q2[:, m * H + h], q[:, h, m])
            assert torch.equal(k2[:, (m * H + h) // (H // G)], k[:, h // (H // G), m])
