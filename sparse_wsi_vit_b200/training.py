"""Training-loop glue for the drop-in encoders, free of any trainer framework.

The reference trains through a PyTorch-Lightning wrapper whose step is
``output = self.network(inputs, coords)`` -> loss on ``output["logits"]``
(src/sparse_wsi_vit/experiments/lightning_wrappers/wsi_attn_wrapper.py:75-110) under DDP, one slide
per rank (experiments/trainer.py:100-106).  The encoders of this package take the same call
(``forward(x, coords=None)``), so the reference's wrapper accepts them by changing one import;
``slide_step`` restates that step for use without Lightning (which is not a dependency of this
package), and ``train_step`` adds the optimiser update, for single-slide and ragged batches.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def slide_step(network, batch, multiclass: bool = True, use_bce_loss: bool = False):
    """Forward + loss of one batch dict {"input", "coords", "label"[, "class_weight"]} exactly as the
    reference's ``_step`` computes it (wsi_attn_wrapper.py:75-110).  ``input`` may be a (B, N, F) tensor
    or, for a ragged batch (``ingest.ragged_collate``), a list of (N_i, F) tensors.  Returns (loss, preds, logits)."""
    inputs, coords, labels = batch["input"], batch.get("coords"), batch["label"]
    if isinstance(inputs, (list, tuple)):
        logits = torch.cat([network(x, None if coords is None else coords[i])["logits"] for i, x in enumerate(inputs)])
    else:
        logits = network(inputs, coords)["logits"]
    if logits.shape[1] == 1:
        logits = logits.squeeze(1)
    if not multiclass and use_bce_loss:
        loss = F.binary_cross_entropy_with_logits(logits, labels.float(), reduction="none")
        preds = (torch.sigmoid(logits) >= 0.5).int()
    else:
        loss = F.cross_entropy(logits, labels, reduction="none")
        preds = torch.argmax(logits, dim=-1)
    if "class_weight" in batch:
        loss = loss * torch.as_tensor(batch["class_weight"], device=loss.device, dtype=loss.dtype)
    return loss.mean(), preds, logits


def train_step(network, optimizer, batch, autocast_dtype=torch.bfloat16, **step_kwargs):
    """One optimisation step (the reference runs its steps under ``bf16-mixed`` autocast,
    configs/deepseek_sparse_attention.py:31,104).  Gradients flow through the attention's backward
    kernels.  Returns the loss as a float."""
    optimizer.zero_grad(set_to_none=True)
    dev_type = next(network.parameters()).device.type
    with torch.autocast(dev_type, dtype=autocast_dtype, enabled=autocast_dtype is not None):
        loss, _, _ = slide_step(network, batch, **step_kwargs)
    loss.backward()
    optimizer.step()
    return float(loss.detach())
