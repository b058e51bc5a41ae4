"""The two tiny Llama configurations the tests use.  They differ in every size and option:
layers, width, heads and groups (grouped 2:1 against multi-query 3:1), head size, feed-forward
width, vocabulary, rope base, the norms' eps, tied against untied output matrix, stored dtypes,
norm weights (all ones against 1 + N(0, 0.1)) and page size."""

TINY_A = dict(
    config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", num_hidden_layers=2,
                hidden_size=64, intermediate_size=128, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                vocab_size=256, max_position_embeddings=128, rms_norm_eps=1e-5, rope_theta=10000.0,
                tie_word_embeddings=True),
    seed=0, norm_noise=0.0, matrix_dtype="bfloat16", page_size=4)

TINY_B = dict(
    config=dict(architectures=["LlamaForCausalLM"], model_type="llama", hidden_act="silu", num_hidden_layers=3,
                hidden_size=96, intermediate_size=224, num_attention_heads=3, num_key_value_heads=1, head_dim=32,
                vocab_size=384, max_position_embeddings=256, rms_norm_eps=1e-6, rope_theta=100000.0,
                tie_word_embeddings=False),
    seed=1, norm_noise=0.1, matrix_dtype="float32", page_size=8)

TINIES = {"tinyA": TINY_A, "tinyB": TINY_B}


def write_tiny(model_dir, tiny, std=0.02):
    import torch
    from vitna_anchor_b200.engine.loading import write_random_model
    write_random_model(model_dir, tiny["config"], tiny["seed"], std=std, norm_noise=tiny["norm_noise"],
                       matrix_dtype=getattr(torch, tiny["matrix_dtype"]))
    return model_dir
