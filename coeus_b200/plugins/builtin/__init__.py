"""The six built-in plugins (whitespace / BPE / WordPiece tokenizers, basic and transformer model
builders, checkpoint loader) under the reference's identities."""
from .loader import BasicLoaderPlugin, CheckpointLoaderPlugin  # noqa: F401
from .model_basic import BasicModel, BasicModelBuilder, BasicModelPlugin  # noqa: F401
from .model_transformer import (TransformerModel, TransformerModelBuilder,  # noqa: F401
                                TransformerModelPlugin)
from .tokenizer_basic import BasicTokenizer, BasicTokenizerPlugin  # noqa: F401
from .tokenizer_bpe import BpeTokenizer, BpeTokenizerPlugin  # noqa: F401
from .tokenizer_wordpiece import WordPieceTokenizer, WordPieceTokenizerPlugin  # noqa: F401
