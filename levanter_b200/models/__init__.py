"""Model families.  Importing this package registers every ``LmConfig`` subclass under its ``type:`` key."""
from . import lm_model  # noqa: F401  (first: the others build on it)
from . import llama, gpt2, mistral, mixtral, gemma, qwen, olmo, gpt2_hyena, gated_deltanet  # noqa: F401,E402
from . import asr_model, whisper  # noqa: F401,E402  (speech: a registry of its own, ``ASRConfig``)
