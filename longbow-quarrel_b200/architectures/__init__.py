from . import fetorax, lavutar, llama, raritar, zoporax  # noqa: F401  (registers LlamaForCausalLM, Fetorax, Lavutar, Raritar and Zoporax)
