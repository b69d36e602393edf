"""One rank of a tensor-parallel engine run (launched by tests/test_tp_gpu.py through
torch.distributed.run). Rank 0 writes the generated tokens as JSON."""
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def main():
    import faulthandler
    # a stuck collective shows up as a stack dump instead of a silent wait
    faulthandler.dump_traceback_later(int(os.environ.get("TP_DUMP_AFTER", "120")), exit=True)
    model_dir, out_path, cases = sys.argv[1], sys.argv[2], json.loads(sys.argv[3])
    tp_path = sys.argv[4] if len(sys.argv) > 4 else "auto"
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    from starter_b200 import Engine, _lib
    if os.environ.get("TP_NO_PDL"):
        _lib.check(_lib.lib.q_set_pdl(0))
    if len(sys.argv) > 5:          # largest world that exchanges inside the projections at 1-8 rows
        _lib.check(_lib.lib.q_set_option(b"peer_in_gemm", int(sys.argv[5])))
    engine = Engine(model_dir, device=f"cuda:{local}", group=dist.group.WORLD, tp_path=tp_path)
    if os.environ.get("TP_NO_GRAPH"):
        from starter_b200.decode import DecodeState
        DecodeState.capture = lambda self: None
    out, paths = [], set()
    for prompt, n in cases:
        out.append(list(engine.generate(prompt, n)))
        paths.add(engine.decode_state.tp_path)
    from starter_b200.ops import device_status
    status = device_status()
    if dist.get_rank() == 0:
        Path(out_path).write_text(json.dumps({"tokens": out, "tp_path": "/".join(sorted(paths)),
                                              "device_status": status}))
    # captured graphs hold NCCL kernels: drop them before the communicator goes away
    engine.decode_state = None
    del engine
    torch.cuda.synchronize()
    dist.barrier()
    import threading
    threading.Timer(20.0, os._exit, [0]).start()      # a stalled teardown must not hang the test
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
