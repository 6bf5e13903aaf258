"""Token shard files, the streaming data loader and the tokenisation pipeline."""
from .tokfile import TokenFileWriter, read_token_file, TOK_MAGIC
from .loader import DataLoader

__all__ = ["TokenFileWriter", "read_token_file", "DataLoader", "TOK_MAGIC"]
