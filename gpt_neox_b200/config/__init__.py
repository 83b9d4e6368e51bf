from .arguments import ATTENTION_TYPE_CHOICES, FIELDS, NeoXArgs, expand_attention_types, gen_docs  # noqa: F401
