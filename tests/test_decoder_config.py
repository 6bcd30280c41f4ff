"""Host-side arithmetic of the synthetic decoder: the bytes a decode step must read."""
from leviathan_b200.decoder import DecoderConfig


def test_bytes_per_token_of_the_30_layer_decoder():
    b = DecoderConfig().bytes_per_token()
    # Q4_0 q [4096 x 2816], k, v [2048 x 2816], o [2816 x 4096]: 18 bytes per 32 values
    assert b["attention_weights"] == (4096 * 2816 + 2 * 2048 * 2816 + 2816 * 4096) // 32 * 18 == 19_464_192
    # one expert: gate_up [1408 x 2816] + down [2816 x 704]
    assert b["expert"] == (1408 * 2816 + 2816 * 704) // 32 * 18 == 3_345_408
    assert b["router"] == 128 * 2816 * 4
    # fp16 K and V of 4096 positions x 8 heads x 256
    assert b["kv_per_sequence"] == 2 * 4096 * 8 * 256 * 2 == 33_554_432
    # Q6_K head [262144 x 2816]: 210 bytes per 256 values
    assert b["head"] == 262144 * 11 * 210 == 605_552_640
    assert b["batch_1_total"] == 30 * (19_464_192 + 1_441_792 + 8 * 3_345_408 + 33_554_432) + 605_552_640
    assert abs(b["batch_1_total"] / 1e9 - 3.04) < 0.01


def test_smaller_shapes_scale():
    c = DecoderConfig(hidden=256, layers=2, q_heads=4, kv_heads=2, head_dim=128, experts=8, top_k=2, expert_inter=64, vocab=512, positions=48)
    b = c.bytes_per_token()
    assert b["head"] == 512 * 1 * 210 and b["kv_per_sequence"] == 2 * 48 * 2 * 128 * 2
