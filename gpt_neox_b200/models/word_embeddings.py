"""Input embeddings (megatron/model/word_embeddings.py:24-251): vocab-parallel word embedding,
optional learned / sinusoidal position embedding, dropout, sequence-parallel scatter along dim 1;
``EmbeddingPipe`` for the layer list; ``SoftEmbedding`` for prompt tuning."""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from .. import parallel as mpu
from ..parallel.mappings import scatter_to_sequence_parallel_region
from .positional_embeddings import SinusoidalPositionalEmbedding


class StableEmbedding(nn.Embedding):
    """Embedding followed by a LayerNorm (parameters under ``norm.``), Xavier-uniform initialised: what the
    reference takes from bitsandbytes for the serial (position / token-type) embeddings when ``use_bnb_optimizer``
    is set (megatron/model/word_embeddings.py:71-81), as a plain module here."""

    def __init__(self, num_embeddings, embedding_dim):
        super().__init__(num_embeddings, embedding_dim)
        self.norm = nn.LayerNorm(embedding_dim)
        nn.init.xavier_uniform_(self.weight)

    def forward(self, ids):
        return self.norm(super().forward(ids))


class Embedding(nn.Module):
    def __init__(self, neox_args, hidden_size, vocab_size, max_sequence_length, embedding_dropout_prob,
                 init_method, num_tokentypes=0, use_pos_emb=True):
        super().__init__()
        self.embedding_module = StableEmbedding if neox_args.use_bnb_optimizer else nn.Embedding
        self.hidden_size, self.init_method, self.num_tokentypes = hidden_size, init_method, num_tokentypes
        self.sequence_parallel = bool(neox_args.sequence_parallel) and mpu.get_model_parallel_world_size() > 1
        self.use_mup = neox_args.use_mup
        self.mup_embedding_mult = neox_args.mup_embedding_mult
        self.mup_rp_embedding_mult = neox_args.mup_rp_embedding_mult
        self.word_embeddings = mpu.VocabParallelEmbedding(neox_args=neox_args, num_embeddings=vocab_size,
                                                          embedding_dim=hidden_size, init_method=init_method)
        self.use_pos_emb = use_pos_emb
        self.embedding_type = neox_args.pos_emb if use_pos_emb else None
        if self.use_pos_emb and self.embedding_type == "learned":
            self.position_embeddings = self.embedding_module(max_sequence_length, hidden_size)
            self.init_method(self.position_embeddings.weight)
            self.opt_pos_emb_offset = neox_args.opt_pos_emb_offset
        elif self.use_pos_emb and self.embedding_type == "sinusoidal":
            self.position_embeddings = SinusoidalPositionalEmbedding(hidden_size)
        if num_tokentypes > 0:
            self.tokentype_embeddings = self.embedding_module(num_tokentypes, hidden_size)
            self.init_method(self.tokentype_embeddings.weight)
        else:
            self.tokentype_embeddings = None
        self.embedding_dropout = nn.Dropout(embedding_dropout_prob)

    def add_tokentype_embeddings(self, num_tokentypes):
        if self.tokentype_embeddings is not None:
            raise Exception("tokentype embeddings is already initialized")
        self.num_tokentypes = num_tokentypes
        self.tokentype_embeddings = self.embedding_module(num_tokentypes, self.hidden_size)
        self.init_method(self.tokentype_embeddings.weight)

    def forward(self, input_ids, position_ids, tokentype_ids=None):
        # sequence parallelism: when nothing between the lookup and the scatter needs the whole sequence, the lookup
        # itself delivers this rank's slice (over peer memory each row goes only to the rank that owns its position)
        pos_table = self.use_pos_emb and self.embedding_type in ("learned", "sinusoidal")
        early = (self.sequence_parallel and not pos_table and tokentype_ids is None
                 and not (self.training and self.embedding_dropout.p > 0))
        embeddings = self.word_embeddings(input_ids, to_sequence_parallel=True) if early else \
            self.word_embeddings(input_ids)
        if self.use_pos_emb and self.embedding_type in ("learned", "sinusoidal"):
            if self.embedding_type == "learned" and self.opt_pos_emb_offset:
                position_ids = position_ids + self.opt_pos_emb_offset
            pe = self.position_embeddings(position_ids)
            if self.use_mup:
                pe = pe * self.mup_rp_embedding_mult
            embeddings = embeddings + pe.to(embeddings.dtype)
        if tokentype_ids is not None:
            embeddings = embeddings + self.tokentype_embeddings(tokentype_ids)
        embeddings = self.embedding_dropout(embeddings)
        if self.use_mup:
            with torch.no_grad():
                embeddings.mul_(self.mup_embedding_mult)
        if self.sequence_parallel and not early:
            embeddings = scatter_to_sequence_parallel_region(embeddings, seq_dim=1)
        return embeddings


class EmbeddingPipe(Embedding):
    """``(input_ids, position_ids, attention_mask)`` -> ``(embeddings, attention_mask)``."""

    @property
    def word_embeddings_weight(self):
        return self.word_embeddings.weight

    def forward(self, args):
        assert len(args) == 3, f"Expected 3 arguments (input_ids, position_ids, attention_mask), but got {len(args)}."
        input_ids, position_ids, attention_mask = args
        return super().forward(input_ids, position_ids), attention_mask


class SoftEmbedding(nn.Module):
    """Learned soft prompt prepended to the embeddings (prompt tuning)."""

    def __init__(self, neox_args, wte, n_tokens: int = 10, init_range: float = 0.5, init_string: str = ""):
        super().__init__()
        self.n_tokens, self.neox_args = n_tokens, neox_args
        self.init_range, self.init_string = init_range, init_string
        self.soft_embedding_weight = nn.Parameter(self.initialize_embedding(wte))

    def initialize_embedding(self, wte=None):
        if self.init_string and wte is not None and getattr(self.neox_args, "tokenizer", None) is not None:
            ids = torch.LongTensor(self.neox_args.tokenizer.tokenize(self.init_string)).to(wte.weight.device)
            emb = wte(ids)
            if emb.shape[0] >= self.n_tokens:
                return emb[: self.n_tokens].detach().clone()
            reps = math.ceil(self.n_tokens / emb.shape[0])
            return emb.repeat(reps, 1)[: self.n_tokens].detach().clone()
        return torch.empty(self.n_tokens, self.neox_args.hidden_size).uniform_(-self.init_range, self.init_range)

    def forward(self, args):
        in_inference = not isinstance(args, tuple) or len(args) == 3
        if isinstance(args, tuple) and len(args) == 3:
            embedding, layer_past, attention_mask = args
        else:
            embedding, attention_mask = args
            layer_past = None
        soft = self.soft_embedding_weight.to(embedding.dtype).repeat(embedding.shape[0], 1, 1)
        # the soft prompt is prepended once, on the first (cache-less) step of a generation
        if layer_past is None or (torch.is_tensor(layer_past) and layer_past.numel() == 0):
            embedding = torch.cat((soft, embedding), dim=1)[:, : self.neox_args.seq_length]
        if in_inference and layer_past is not None:
            return embedding, layer_past, attention_mask
        return embedding, attention_mask
