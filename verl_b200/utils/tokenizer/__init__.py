from .tokenizer import hf_processor, hf_tokenizer, set_pad_token_id  # noqa: F401
