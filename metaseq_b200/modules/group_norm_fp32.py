"""GroupNorm evaluated in fp32 whatever the activation dtype (reference: metaseq/modules/group_norm_fp32.py)."""
from __future__ import annotations

import torch.nn as nn
import torch.nn.functional as F


class GroupNormFp32(nn.GroupNorm):
    def forward(self, input):
        w = None if self.weight is None else self.weight.float()
        b = None if self.bias is None else self.bias.float()
        return F.group_norm(input.float(), self.num_groups, w, b, self.eps).type_as(input)
