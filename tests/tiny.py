"""Tiny configurations of the Qwen2 decoder for the tests. They differ in every size and
option: head counts and groups, sizes that are no power of two, layers, vocabulary, eps,
rope base, tied or untied head, an explicit head size, the window, and the head sizes that
the different attention kernels take."""
import torch

_BASE = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_act": "silu"}

TINY = {
    # 2 layers, 4 heads in 2 groups, head size 16, tied head, every key visible
    "A": dict(_BASE, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, vocab_size=256, max_position_embeddings=128, rms_norm_eps=1e-6,
              rope_theta=10000.0, tie_word_embeddings=True, eos_token_id=255),
    # 3 layers, 3 heads on 1 kv head, head size 32, untied head, layers 1.. see a window of 40
    "B": dict(_BASE, hidden_size=96, intermediate_size=160, num_hidden_layers=3, num_attention_heads=3,
              num_key_value_heads=1, vocab_size=384, max_position_embeddings=96, rms_norm_eps=1e-5,
              rope_theta=1000000.0, tie_word_embeddings=False, use_sliding_window=True, sliding_window=40,
              max_window_layers=1),
    # long contexts: width and vocabulary no power of two, head size given and not width/heads,
    # as many kv heads as heads, a window of 100 (its ring of 128 positions wraps around)
    "C": dict(_BASE, hidden_size=80, intermediate_size=208, num_hidden_layers=2, num_attention_heads=5,
              num_key_value_heads=5, head_dim=48, vocab_size=300, max_position_embeddings=2048,
              rms_norm_eps=3e-6, rope_theta=50000.0, tie_word_embeddings=True, use_sliding_window=True,
              sliding_window=100, max_window_layers=1),
    # head size 64 (the size the tcgen05 prefill attention takes), 6 heads on 3 kv heads, bias-free rotary base,
    # untied head, a context long enough for prompts of several key tiles and decoding over several chunks
    "D": dict(_BASE, hidden_size=384, intermediate_size=272, num_hidden_layers=2, num_attention_heads=6,
              num_key_value_heads=3, vocab_size=331, max_position_embeddings=4096, rms_norm_eps=1e-5,
              rope_theta=500000.0, tie_word_embeddings=False),
    # head size 128 (the larger tile of the tcgen05 attention, the fused q/k/v epilogue and the decode kernel's
    # tensor-map path), given and not width/heads; width, feed-forward and vocabulary no power of two
    "E": dict(_BASE, hidden_size=264, intermediate_size=344, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=2, head_dim=128, vocab_size=515, max_position_embeddings=1024, rms_norm_eps=2e-6,
              rope_theta=250000.0, tie_word_embeddings=False),
}
SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3, "E": 4}

# The layer sizes of Qwen2.5-0.5B (width 896, 14 heads on 2 kv heads of 64, feed-forward 4864, vocabulary 151,936,
# tied head) with 2 of its 24 layers: what the kernels see at a real size, small enough for the plain model on the CPU.
REAL_0_5B_2_LAYERS = dict(_BASE, hidden_size=896, intermediate_size=4864, num_hidden_layers=2, num_attention_heads=14,
                          num_key_value_heads=2, vocab_size=151936, max_position_embeddings=32768, rms_norm_eps=1e-6,
                          rope_theta=1000000.0, tie_word_embeddings=True)


def make_model_dir(name: str, path: str) -> str:
    from smolmoe_c99_b200.config import config_from_json
    from smolmoe_c99_b200.weights import write_random_model

    return write_random_model(config_from_json(TINY[name]), path, SEEDS[name])


def random_tokens(n: int, vocab: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
