"""The tiny configurations the tests use.  They differ in every size and option."""

TINY_A = dict(architecture="mqa_gpt", vocab_size=256, d_model=64, num_layers=2, num_heads=4, num_kv_heads=1,
              hidden_size=176, max_seq_len=64, rope_theta=10000.0, rms_norm_eps=1e-5, bias=False,
              eos_token_id=255, dtype="float32")
TINY_B = dict(architecture="mqa_gpt", vocab_size=1000, d_model=96, num_layers=3, num_heads=3, num_kv_heads=1,
              hidden_size=256, max_seq_len=128, rope_theta=500000.0, rms_norm_eps=1e-6, bias=True,
              eos_token_id=999, dtype="float32")
# grouped kv heads, a long context for page reuse and far keys, head size 48 (a step of 16, no power of two)
TINY_C = dict(architecture="mqa_gpt", vocab_size=515, d_model=288, num_layers=2, num_heads=6, num_kv_heads=2,
              hidden_size=200, max_seq_len=640, rope_theta=20000.0, rms_norm_eps=3e-6, bias=False,
              eos_token_id=None, dtype="float32")

SEEDS = {"A": 11, "B": 23, "C": 37}
PAGE = {"A": 16, "B": 8, "C": 32}
