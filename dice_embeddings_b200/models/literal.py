"""Literal (numeric attribute) regression head on top of entity embeddings.

``(entity, data property) → value``: concatenated embeddings → Linear → LayerNorm → ReLU → Dropout, a gated
residual projection, then a scalar output.  Parameter names (``data_property_embeddings``, ``fc``, ``fc_out``,
``gated_residual_proj``, ``layer_norm``) are the keys of ``literal_model.pt``
(reference ``dicee/models/literal.py:5-89``).
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class LiteralEmbeddings(nn.Module):
    def __init__(self, num_of_data_properties: int, embedding_dims: int, entity_embeddings: nn.Embedding,
                 dropout: float = 0.3, gate_residual: bool = True, freeze_entity_embeddings: bool = True):
        super().__init__()
        self.embedding_dim = embedding_dims
        self.num_of_data_properties = num_of_data_properties
        self.hidden_dim = embedding_dims * 2
        self.gate_residual = gate_residual
        self.freeze_entity_embeddings = freeze_entity_embeddings
        self.entity_embeddings = nn.Embedding.from_pretrained(entity_embeddings.weight.detach().clone(),
                                                              freeze=freeze_entity_embeddings)
        self.data_property_embeddings = nn.Embedding(num_of_data_properties, self.embedding_dim)
        self.fc = nn.Linear(self.hidden_dim, self.hidden_dim)
        self.fc_out = nn.Linear(self.hidden_dim, 1)
        self.dropout = nn.Dropout(p=dropout)
        self.gated_residual_proj = nn.Linear(self.hidden_dim * 2, self.hidden_dim * 2)
        self.layer_norm = nn.LayerNorm(self.hidden_dim)

    def forward(self, entity_idx: torch.Tensor, attr_idx: torch.Tensor) -> torch.Tensor:
        pair = torch.cat((self.entity_embeddings(entity_idx), self.data_property_embeddings(attr_idx)), dim=1)
        z = self.dropout(F.relu(self.layer_norm(self.fc(pair))))
        if self.gate_residual:
            value, gate = self.gated_residual_proj(torch.cat((z, pair), dim=1)).chunk(2, dim=-1)
            residual = value * torch.sigmoid(gate)
        else:
            residual = z + pair
        return self.fc_out(residual).flatten()

    @property
    def device(self):
        return next(self.parameters()).device
