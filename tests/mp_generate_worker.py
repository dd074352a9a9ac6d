"""Worker of the 2-GPU generation test (one process per GPU, launched by torchrun): greedy
generation with KV heads sharded over the ranks - eager (NCCL all-gather per layer) and recorded
(CUDA graph with the fused peer gather) - against the un-sharded run on the same GPU."""

from __future__ import annotations

import os
import sys
import warnings

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


class StubTokenizer:
    eos_token_id = None

    def decode(self, ids, skip_special_tokens=True):
        return " ".join(str(int(i)) for i in ids)

    def encode(self, text, add_special_tokens=False):
        return [int(t) for t in text.split()]


def main() -> None:
    from transformers import LlamaConfig, LlamaForCausalLM

    import turboquant
    from tq_local_b200.runtime.sharding import HeadShard

    rank = int(os.environ["RANK"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=512)
    model = LlamaForCausalLM(cfg).eval().to(dev, torch.bfloat16)
    ids = torch.randint(0, 512, (2, 40), generator=torch.Generator().manual_seed(3)).to(dev)
    new = 20

    def run(**kw):
        turboquant.activate(model, StubTokenizer(), quiet=True, bits=4, verify=False, **kw)
        try:
            return model.generate(ids, max_new_tokens=new)
        finally:
            turboquant.deactivate(model, quiet=True)

    whole = run(cuda_graph=False)
    shard = HeadShard.from_process_group()
    eager = run(shard=shard, cuda_graph=False)
    with warnings.catch_warnings():
        warnings.simplefilter("error")  # the sharded step must record
        recorded = run(shard=shard, cuda_graph=True)
    for name, got in (("eager", eager), ("recorded", recorded)):
        assert tuple(got.shape) == (2, 40 + new), name
        assert torch.equal(got[:, :42], whole[:, :42]), name
        assert (got == whole).float().mean() >= 0.9, name
    both = [torch.empty_like(recorded) for _ in range(2)]
    dist.all_gather(both, recorded)
    assert torch.equal(both[0], both[1])  # the ranks agree on every token
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("GENERATE_OK")


if __name__ == "__main__":
    main()
