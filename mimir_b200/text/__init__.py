"""Text models (reference: text/): a WordPiece tokenizer (BERT's uncased rules), vocabularies built from
texts, the BERT encoder with masked-LM and classification heads, and a classifier of token ids that hides
padding and swaps heads."""
from .wordpiece import WordPiece, build_vocab  # noqa: F401
from .bert import Bert, BertConfig, BertForMaskedLM, BertForSequenceClassification, TextClassifier  # noqa: F401
