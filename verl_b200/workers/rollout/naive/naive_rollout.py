"""In-process generation without the serving engine: a plain batched decode loop over the model's own forward, with a
dense (non-paged) KV cache rebuilt from the packed forward each step on CPU-sized problems.

``NaiveRollout.generate_sequences(DataProto)`` has the same batch contract as the engine-backed worker method: left
padded ``input_ids / attention_mask / position_ids`` in; ``prompts, responses, input_ids, attention_mask, position_ids,
response_mask, rollout_log_probs`` out. It recomputes the whole prefix every step (O(L²)), so it is a correctness
oracle and a fallback for tiny models, not a serving path (reference: ``verl/workers/rollout/naive/naive_rollout.py``
and ``hf_rollout.py:39-177`` — ``module.generate`` under ``summon_full_params``).
"""

from __future__ import annotations

import torch

from verl_b200.models.transformer import DecoderLM, PackedBatch
from verl_b200.protocol import DataProto, TensorBatch
from verl_b200.utils.torch_functional import compute_position_id_with_mask

__all__ = ["NaiveRollout", "HFRollout"]


class NaiveRollout:
    def __init__(self, model: DecoderLM, response_length: int = 64, temperature: float = 1.0, top_k: int = -1, do_sample: bool = True,
                 micro_batch_size: int = 16):
        self.model, self.response_length, self.temperature, self.top_k, self.do_sample = model, response_length, temperature, top_k, do_sample
        self.micro_batch_size = micro_batch_size

    @torch.no_grad()
    def _next_logits(self, seqs: list[list[int]]) -> torch.Tensor:
        dev = next(self.model.parameters()).device
        lens = torch.tensor([len(s) for s in seqs], dtype=torch.int32)
        cu = torch.zeros(len(seqs) + 1, dtype=torch.int32)
        cu[1:] = torch.cumsum(lens, 0)
        ids = torch.tensor([t for s in seqs for t in s], dtype=torch.int64, device=dev)
        pos = torch.cat([torch.arange(int(n), dtype=torch.int32) for n in lens]).to(dev)
        h = self.model.forward_hidden(PackedBatch(ids, pos, cu.to(dev), cu, int(lens.max())))
        last = (cu[1:] - 1).long().to(dev)
        return torch.nn.functional.linear(h.index_select(0, last), self.model.output_weight).float()

    @torch.no_grad()
    def generate_sequences(self, prompts: DataProto) -> DataProto:
        ids, att = prompts.batch["input_ids"].cpu(), prompts.batch["attention_mask"].cpu().bool()
        meta = prompts.meta_info
        eos = meta.get("eos_token_id")
        eos_ids = set() if eos is None else ({eos} if isinstance(eos, int) else set(eos))
        pad = int(meta.get("pad_token_id", 0) or 0)
        R = int(meta.get("response_length", self.response_length))
        do_sample = bool(meta.get("do_sample", self.do_sample))
        temperature = float(meta.get("temperature", self.temperature))
        gen = torch.Generator().manual_seed(int(meta.get("seed", 0)))
        bs, P = ids.shape
        seqs = [ids[i][att[i]].tolist() for i in range(bs)]
        out_tok = [[] for _ in range(bs)]
        out_lp = [[] for _ in range(bs)]
        live = list(range(bs))
        for _ in range(R):
            if not live:
                break
            logits = torch.cat([self._next_logits([seqs[i] + out_tok[i] for i in live[s: s + self.micro_batch_size]]).cpu()
                                for s in range(0, len(live), self.micro_batch_size)])
            if do_sample and temperature > 0:
                logits = logits / temperature
                if self.top_k > 0:
                    kth = logits.topk(self.top_k, -1).values[:, -1:]
                    logits = logits.masked_fill(logits < kth, float("-inf"))
                logp = torch.log_softmax(logits, -1)
                tok = torch.multinomial(logp.exp(), 1, generator=gen)[:, 0]
            else:
                logp = torch.log_softmax(logits, -1)
                tok = logp.argmax(-1)
            nxt = []
            for row, i in enumerate(live):
                t = int(tok[row])
                out_tok[i].append(t)
                out_lp[i].append(float(logp[row, t]))
                if t not in eos_ids:
                    nxt.append(i)
            live = nxt
        resp = torch.full((bs, R), pad, dtype=ids.dtype)
        rmask = torch.zeros(bs, R, dtype=torch.int64)
        lps = torch.zeros(bs, R)
        for i in range(bs):
            n = len(out_tok[i])
            resp[i, :n] = torch.tensor(out_tok[i], dtype=ids.dtype)
            rmask[i, :n] = 1
            lps[i, :n] = torch.tensor(out_lp[i])
        full_att = torch.cat([att.long(), rmask], 1)
        batch = TensorBatch({"prompts": ids, "responses": resp, "input_ids": torch.cat([ids, resp], 1), "attention_mask": full_att,
                             "position_ids": compute_position_id_with_mask(full_att), "response_mask": rmask, "rollout_log_probs": lps}, batch_size=(bs,))
        return DataProto(batch=batch, non_tensor_batch=dict(prompts.non_tensor_batch), meta_info={})


HFRollout = NaiveRollout
