from . import fetorax, llama, zoporax  # noqa: F401  (registers LlamaForCausalLM, Fetorax and Zoporax)
