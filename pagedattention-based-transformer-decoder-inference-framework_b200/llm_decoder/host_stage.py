"""Host -> device staging of the small integer tensors that describe a step (batch rows, work lists, page-table
updates)."""
import torch


class _PinnedStage:
    """A pinned int32 staging buffer per device for the small host tensors that describe a step.  Pieces are packed one
    after the other and copied with asynchronous copies, so building a step's description never waits for the GPU (a copy
    from pageable memory synchronises with the stream, a freshly pinned buffer per tensor costs a host allocation each).
    A region is reused only after a wrap-around, which first waits for the stream: every copy out of it has run by then."""
    CAPACITY = 4 << 20          # int32 elements

    def __init__(self):
        self.buf = torch.empty(self.CAPACITY, dtype=torch.int32).pin_memory()
        self.off = 0

    def put(self, t, device):
        n = t.numel()
        if t.dtype != torch.int32 or n == 0 or n > self.CAPACITY // 4:
            return t.to(device)
        if self.off + n > self.CAPACITY:
            torch.cuda.current_stream(device).synchronize()
            self.off = 0
        view = self.buf[self.off:self.off + n].view(t.shape)
        view.copy_(t)
        self.off += (n + 3) // 4 * 4
        return view.to(device, non_blocking=True)


_STAGES = {}


def to_device(t, device):
    """A small host tensor of one step's batch description onto the device."""
    if device.type != "cuda":
        return t
    stage = _STAGES.get(device)
    if stage is None:
        stage = _STAGES[device] = _PinnedStage()
    return stage.put(t.contiguous(), device)
