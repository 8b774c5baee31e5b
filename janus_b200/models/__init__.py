from . import llama, zivitar  # noqa: F401  (registers LlamaForCausalLM and Zivitar)
