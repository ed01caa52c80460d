from . import fetorax, llama, raritar, zoporax  # noqa: F401  (registers LlamaForCausalLM, Fetorax, Raritar and Zoporax)
