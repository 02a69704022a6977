"""Command line in the manner of the reference's qwen3_chat, chat template and tokenizer."""
