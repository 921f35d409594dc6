"""Two-stage pipeline parallelism with a hand-written 1F1B schedule.

Stage 0 holds the embedding and the first half of the blocks, stage 1 the second half, final norm
and LM head (`GPT(stage_index=...)`).  The reference builds this on
`torch.distributed.pipelining.Schedule1F1B` (`runtime/pipeline.py:14-120`); here the schedule is
explicit: micro-batches are the gradient-accumulation steps, stage 0 runs one forward ahead, and in
the steady state each stage exchanges "activation forward / gradient backward" as one batched
isend/irecv pair so neither side can block the other.  The MoE balance loss of stage 0 travels with
the activations and its gradient travels back.  Works over NCCL (GPUs) and gloo (CPU tests).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor


class PipelineRuntime:
    def __init__(self, model, rank: int, world_size: int, device: str, grad_accum_mini_steps: int,
                 use_doc_masking: bool) -> None:
        assert world_size == 2, "the pipeline has exactly two stages"
        self.model, self.rank, self.device = model, rank, device
        self.master_process = rank == 0
        self.accum = grad_accum_mini_steps
        self.use_doc_masking = use_doc_masking
        self.hidden = model.gpt_config.hidden_size
        self.has_balance = model.gpt_config.use_moe and model.moe_load_balance_weight > 0

    # ---- data ---------------------------------------------------------------------------------------
    def next_batch(self, data_loader, batch_size: int, seq_len: int) -> Tuple[Optional[Tensor], Tensor, Optional[Tensor]]:
        """Rank 0 owns the loader; targets and document ids are broadcast (reference `runtime/pipeline.py:56-72`)."""
        if self.master_process:
            x, y, docs = data_loader.next_batch()
            x, y = x[:batch_size].to(self.device), y[:batch_size].to(self.device)
            docs = docs[:batch_size].to(self.device) if docs is not None else None
        else:
            x = None
            y = torch.empty((batch_size, seq_len), dtype=torch.long, device=self.device)
            docs = torch.empty((batch_size, seq_len), dtype=torch.int32, device=self.device) if self.use_doc_masking else None
        dist.broadcast(y, src=0)
        if docs is not None:
            dist.broadcast(docs, src=0)
        return x, y, docs

    # ---- point-to-point helpers -------------------------------------------------------------------------
    def _exchange(self, send: List[Tensor], recv: List[Tensor], peer: int) -> None:
        ops = [dist.P2POp(dist.isend, t.contiguous(), peer) for t in send] + [dist.P2POp(dist.irecv, t, peer) for t in recv]
        if ops:
            for work in dist.batch_isend_irecv(ops):
                work.wait()

    def _act_buffers(self, batch: int, seq: int, dtype) -> List[Tensor]:
        bufs = [torch.empty((batch, seq, self.hidden), dtype=dtype, device=self.device)]
        if self.has_balance:
            bufs.append(torch.empty((), dtype=torch.float32, device=self.device))
        return bufs

    # ---- training ------------------------------------------------------------------------------------------
    def train_step(self, batches: List[Tuple[Optional[Tensor], Tensor, Optional[Tensor]]]) -> Tensor:
        """One optimizer step's worth of micro-batches under 1F1B.  Returns [loss, token_loss, balance_term]
        averaged over micro-batches on the last stage and zeros on the first."""
        m = len(batches)
        scale = 1.0 / m
        act_dtype = torch.float32
        losses = torch.zeros(3, device=self.device)
        if self.rank == 0:
            pending: List[Tuple[Tensor, Optional[Tensor]]] = []

            def forward(i: int) -> List[Tensor]:
                x, _, docs = batches[i]
                out = self.model(x, document_ids=docs)
                act, bal = out if isinstance(out, tuple) else (out, None)
                pending.append((act, bal))
                send = [act.detach().to(act_dtype)]
                if self.has_balance:
                    send.append((bal if bal is not None else act.new_zeros(())).detach().float())
                return send

            def backward(grads: List[Tensor]) -> None:
                act, bal = pending.pop(0)
                tensors, gs = [act], [grads[0].to(act.dtype)]
                if self.has_balance and bal is not None:
                    tensors.append(bal)
                    gs.append(grads[1].to(bal.dtype))
                torch.autograd.backward(tensors, gs)

            b, t = batches[0][0].shape
            self._exchange(forward(0), [], 1)                                    # warm-up: one forward ahead
            for i in range(1, m):
                grads = self._act_buffers(b, t, act_dtype)
                self._exchange(forward(i), grads, 1)                             # send activation i, receive gradient i-1
                backward(grads)
            grads = self._act_buffers(b, t, act_dtype)
            self._exchange([], grads, 1)                                         # cool-down
            backward(grads)
        else:
            b, t = batches[0][1].shape
            incoming = self._act_buffers(b, t, act_dtype)
            self._exchange([], incoming, 0)
            for i in range(m):
                _, y, docs = batches[i]
                act = incoming[0].requires_grad_()
                bal = incoming[1].requires_grad_() if self.has_balance else None
                loss, token_loss, balance = self.model(act, y, document_ids=docs, previous_stage_balance_loss=bal)
                (loss * scale).backward()
                losses += torch.stack((loss.detach().float(), token_loss.detach().float(), balance.detach().float())) * scale
                outgoing = [act.grad] + ([bal.grad if bal.grad is not None else torch.zeros_like(bal)] if self.has_balance else [])
                incoming = self._act_buffers(b, t, act_dtype) if i + 1 < m else []
                self._exchange(outgoing, incoming, 0)                            # send gradient i, receive activation i+1
        return losses

    # ---- forward only ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def non_training_forward(self, model, indices: Optional[Tensor], targets: Optional[Tensor] = None,
                             attn_mask: Optional[Tensor] = None, ignore_doc_mask: bool = False,
                             document_ids: Optional[Tensor] = None) -> Optional[Tensor]:
        """Stage 0 runs its half and sends the activations; stage 1 finishes and returns loss or logits
        (reference `runtime/pipeline.py:97-120`).  Shapes are sent first because evaluation batches vary."""
        if self.master_process:
            out = model(indices, attn_mask=attn_mask, ignore_doc_mask=ignore_doc_mask, document_ids=document_ids)
            x = out[0] if isinstance(out, tuple) else out
            meta = [(tuple(x.shape), x.dtype)]
            dist.broadcast_object_list(meta, src=0)
            dist.send(x.contiguous(), dst=1)
            return torch.zeros((), device=self.device) if targets is not None else None
        meta = [None]
        dist.broadcast_object_list(meta, src=0)
        shape, dtype = meta[0]
        x = torch.empty(shape, dtype=dtype, device=self.device)
        dist.recv(x, src=0)
        return model(x, targets, attn_mask=attn_mask, ignore_doc_mask=ignore_doc_mask, document_ids=document_ids)
