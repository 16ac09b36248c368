"""Fire-and-forget agent loops that deliver finished trajectories into the TransferQueue
(reference: ``verl/trainer/ppo/v1/agent_loop_tq.py:53-233``)."""

from __future__ import annotations

import asyncio
import threading
from typing import Optional

import numpy as np

from verl_b200.experimental.agent_loop.agent_loop import AgentLoopWorker
from verl_b200.protocol import DataProto
from verl_b200.utils.transfer_queue import KVBatchMeta, TransferQueue, get_transfer_queue

__all__ = ["AgentLoopManagerTQ"]


class AgentLoopManagerTQ:
    """``submit(prompts, gen_step)`` returns at once; a background event loop runs one task per trajectory and writes
    each result under key ``"{uid}#{j}"`` with tags ``{uid, status, gen_step, score}`` as soon as it is done."""

    def __init__(self, config, server_manager, tokenizer, tools=None, reward_fn=None, tq: Optional[TransferQueue] = None,
                 partition_id: str = "train"):
        self.tq = tq or get_transfer_queue()
        self.partition_id = partition_id
        self.server_manager = server_manager
        self.worker = AgentLoopWorker(config, server_manager.client(), tokenizer, tools, reward_fn)
        self._loop = asyncio.new_event_loop()
        self._thread = threading.Thread(target=self._run_loop, name="agent-loop-tq", daemon=True)
        self._thread.start()
        self.inflight = 0
        self._lock = threading.Lock()

    def _run_loop(self):
        asyncio.set_event_loop(self._loop)
        self._loop.run_forever()

    async def _one(self, key: str, uid: str, row: DataProto, gen_step: int):
        self.tq.kv_put(self.partition_id, key, tags={"uid": uid, "status": "running", "gen_step": gen_step})
        try:
            out = await self.worker.generate_sequences_async(row)
            score = float(out.batch["rm_scores"].sum()) if "rm_scores" in out.batch.keys() else None
            out.non_tensor_batch["uid"] = np.array([uid], dtype=object)
            self.tq.kv_batch_put(KVBatchMeta(self.partition_id, [key]), out, tags={"status": "finished", "score": score})
        except Exception as e:  # noqa: BLE001 - the group is evicted by the replay buffer
            self.tq.kv_put(self.partition_id, key, tags={"status": "failure", "error": repr(e)})
        finally:
            with self._lock:
                self.inflight -= 1

    def submit(self, prompts: DataProto, gen_step: int, n: int = 1) -> list[str]:
        """``prompts`` has one row per prompt (with ``uid``); every prompt is rolled out ``n`` times."""
        keys = []
        self.server_manager.wake_up()
        for i in range(len(prompts)):
            uid = str(prompts.non_tensor_batch["uid"][i])
            row = prompts[i: i + 1]
            row.meta_info = dict(prompts.meta_info)
            for j in range(n):
                key = f"{uid}#{j}"
                r = DataProto(batch=row.batch, non_tensor_batch=dict(row.non_tensor_batch), meta_info={**row.meta_info, "seed": int(row.meta_info.get("seed", 0)) * 1000 + 7919 * j + i})
                self.tq.kv_put(self.partition_id, key, tags={"uid": uid, "status": "pending", "gen_step": gen_step})
                with self._lock:
                    self.inflight += 1
                asyncio.run_coroutine_threadsafe(self._one(key, uid, r, gen_step), self._loop)
                keys.append(key)
        return keys

    def abort(self):
        """Interrupt generation (weight update ahead); resumable clients continue the partial trajectories afterwards."""
        self.server_manager.abort_all_requests()

    def shutdown(self, timeout_s: float = 60.0):
        """Stop resuming, interrupt what is running, wait for the tasks to report, then stop the event loop."""
        import time

        self.worker.client.closed = True
        t0 = time.time()
        while self.inflight > 0 and time.time() - t0 < timeout_s:
            self.server_manager.abort_all_requests()
            time.sleep(0.01)
        try:        # close the HTTP session of remote replicas inside its own event loop
            asyncio.run_coroutine_threadsafe(self.worker.client.close(), self._loop).result(timeout=5)
        except Exception:  # noqa: BLE001 - best effort at shutdown
            pass
        self._loop.call_soon_threadsafe(self._loop.stop)
        self._thread.join(timeout=10)
