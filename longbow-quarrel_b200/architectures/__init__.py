from . import fetorax, llama  # noqa: F401  (registers LlamaForCausalLM and Fetorax)
