"""The two tiny TinyGPT configurations of the tests; they differ in every size and option."""
TINY_A = dict(architectures=["GPT2LMHeadModel"], model_type="gpt2", n_layer=2, n_embd=64, n_head=2, n_inner=256,
              vocab_size=256, n_positions=128, activation_function="gelu_new", layer_norm_epsilon=1e-5,
              tie_word_embeddings=True)
TINY_B = dict(architectures=["TinyGPT"], n_layer=3, n_embd=96, n_head=4, n_inner=320, vocab_size=317,
              n_positions=96, activation_function="gelu", layer_norm_epsilon=1e-6, tie_word_embeddings=False)
# standard deviations of the random weights: matrices, biases, norm weights, norm biases
INIT_A = (0.02, 0.0, 0.0, 0.0)
INIT_B = (0.05, 0.02, 0.1, 0.1)
PAGE_A, PAGE_B = 16, 8
