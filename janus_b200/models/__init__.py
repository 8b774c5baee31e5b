from . import llama, ramolix, zivitar  # noqa: F401  (registers LlamaForCausalLM, Ramolix and Zivitar)
