"""The caller of the LookupFFN path: the prenorm RoBERTa encoder whose feed-forward blocks are LookupFFN
layers (reference: src/roberta/models/prenorm_lookup/layer.py:10-78, encoder.py:9-37, and RobertaEmbeddings,
src/roberta/models/postnorm.py:6-28).  Module and parameter names follow the reference, so its checkpoints
load with strict=True.  Attention is ordinary library code (torch scaled_dot_product_attention); only the FFN
runs on this package's kernels.
"""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .lookup import LookupFFN


class RobertaEmbeddings(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.pad_token_id = config.pad_token_id
        self.word_embeddings = nn.Embedding(config.vocab_size, config.hidden_size)
        self.position_embeddings = nn.Embedding(config.max_position_embeddings + 2, config.hidden_size)
        self.token_type_embeddings = nn.Embedding(config.type_vocab_size, config.hidden_size)
        self.LayerNorm = nn.LayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.dropout = nn.Dropout(config.hidden_dropout_prob)

    def forward(self, input_ids, token_type_ids, position_ids):
        e = (self.word_embeddings(input_ids) + self.token_type_embeddings(token_type_ids)
             + self.position_embeddings(self.pad_token_id + 1 + position_ids))
        return self.dropout(self.LayerNorm(e))


class Attention(nn.Module):
    """Prenorm multi-head self-attention (reference layer.py:10-64): softmax(q k^T / sqrt(d_h) - 1000 (1 - mask)) v."""

    def __init__(self, config):
        super().__init__()
        self.num_attention_heads = config.num_attention_heads
        self.attention_head_size = config.attention_head_size
        self.all_head_size = self.num_attention_heads * self.attention_head_size
        self.dropout_p = config.attention_probs_dropout_prob
        self.LayerNorm = nn.LayerNorm(config.hidden_size, eps=config.layer_norm_eps)
        self.query = nn.Linear(config.hidden_size, config.hidden_size)
        self.key = nn.Linear(config.hidden_size, config.hidden_size)
        self.value = nn.Linear(config.hidden_size, config.hidden_size)
        self.dense = nn.Linear(config.hidden_size, config.hidden_size)

    def _heads(self, x):
        b, s, _ = x.shape
        return x.view(b, s, self.num_attention_heads, self.attention_head_size).permute(0, 2, 1, 3)

    def forward(self, hidden_states, attention_mask):
        h = self.LayerNorm(hidden_states)
        q, k, v = self._heads(self.query(h)), self._heads(self.key(h)), self._heads(self.value(h))
        bias = (-1000.0 * (1.0 - attention_mask[:, None, None, :].to(q.dtype)))
        ctx = F.scaled_dot_product_attention(q, k, v, attn_mask=bias,
                                             dropout_p=self.dropout_p if self.training else 0.0,
                                             scale=1.0 / math.sqrt(self.attention_head_size))
        b, _, s, _ = ctx.shape
        return self.dense(ctx.permute(0, 2, 1, 3).reshape(b, s, self.all_head_size))


class EncoderLayer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.FFN = LookupFFN(config, self.hidden_size)
        self.attention = Attention(config)
        self.dropout = nn.Dropout(p=config.hidden_dropout_prob)

    def forward(self, hidden_states, attention_mask):
        attn_output = self.dropout(self.attention(hidden_states, attention_mask)) + hidden_states
        if not self.training or self.dropout.p == 0:
            # dropout is the identity: LayerNorm -> hash -> gather -> + bias -> + residual run as two kernels
            return self.FFN(attn_output, residual=attn_output)
        return self.dropout(self.FFN(attn_output)) + attn_output


class Encoder(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.layer = nn.ModuleList([EncoderLayer(config) for _ in range(config.num_hidden_layers)])
        self.LayerNorm = nn.LayerNorm(config.hidden_size, eps=config.layer_norm_eps)

    def forward(self, hidden_states, attention_mask):
        for layer_module in self.layer:
            hidden_states = layer_module(hidden_states, attention_mask)
        return self.LayerNorm(hidden_states)


class Lookup(nn.Module):
    """`config.encoder_type = "lookupffn_b200.encoder.Lookup"` selects this encoder in a reference config."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.embeddings = RobertaEmbeddings(config)
        self.encoder = Encoder(config)

    def forward(self, input_ids, token_type_ids, position_ids, attention_mask, **kwargs):
        embedding_output = self.embeddings(input_ids, token_type_ids, position_ids)
        return self.encoder(embedding_output, attention_mask), {}

    def get_input_embeddings(self):
        return self.embeddings.word_embeddings

    def set_input_embeddings(self, value):
        self.embeddings.word_embeddings = value
