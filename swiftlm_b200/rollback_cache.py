"""Host-side mirror of the reference's rollback cache for gated-delta (recurrent) layers:
`RecurrentRollbackCache`, Sources/DFlash/RecurrentRollbackCache.swift:34-182 of the SwiftLM
tree, and its protocol `DFlashRollbackCache` (:12-18).

Same method names (snake_case) and the same indexing contract:
  * arm_rollback snapshots [conv_state, recurrent_state] by reference (:63-71);
  * record_tape keeps (tape, k, g, qkv) by reference (:75-85);
  * rollback(n_accepted) restores the snapshot, replays accepted_steps = n_accepted + 1 steps of
    the tape (:115-125) and rebuilds the conv window as
    concat(conv_snapshot, qkv)[:, accepted_steps : accepted_steps + keep] with
    keep = conv_kernel_size - 1 (:139-158);
  * clear_transients drops tape and snapshot (:163-170).
The replay itself runs in libdflash_cuda (tape_replay_kernel).  Unlike the reference, the
accepted length may also be a per-sequence device tensor, in which case nothing is read back to
the host: the replay takes n_per_seq and the conv window is gathered with device indices.
"""
from __future__ import annotations

from typing import List, Optional, Union

import torch

from . import kernels

DEFAULT_CONV_KERNEL_SIZE = 4   # RecurrentRollbackCache.defaultConvKernelSize (:135)


class RecurrentRollbackCache:
    def __init__(self, conv_kernel_size: int = DEFAULT_CONV_KERNEL_SIZE):
        self.conv_kernel_size = conv_kernel_size
        self.state: List[Optional[torch.Tensor]] = [None, None]   # [conv window, recurrent state]
        self.offset = 0
        self._armed = False
        self._tape = self._tape_k = self._tape_g = self._tape_qkv = None
        self._snapshot: Optional[List[Optional[torch.Tensor]]] = None

    # -- arming and recording (:63-88) --
    @property
    def is_armed(self) -> bool:
        return self._armed

    def arm_rollback(self, prefix_len: int = 0) -> None:
        self._armed = True
        self._tape = self._tape_k = self._tape_g = self._tape_qkv = None
        self._snapshot = [self.state[0], self.state[1]]

    def record_tape(self, tape, k, g, qkv) -> None:
        self._tape, self._tape_k, self._tape_g, self._tape_qkv = tape, k, g, qkv

    # -- rollback (:95-131) --
    def rollback(self, n_accepted: Union[int, torch.Tensor]) -> None:
        snapshot = self._snapshot
        if snapshot is None:
            self.clear_transients()
            return
        if snapshot[0] is not None:
            self.state[0] = snapshot[0]
        if snapshot[1] is not None:
            self.state[1] = snapshot[1]
        if self._tape is not None and self._tape_k is not None and self._tape_g is not None and self.state[1] is not None:
            if isinstance(n_accepted, torch.Tensor):
                steps = n_accepted.to(torch.int32) + 1                      # per sequence, stays on the device
                self.state[1] = kernels.tape_replay_kernel(self._tape, self._tape_k, self._tape_g, self.state[1],
                                                           n_per_seq=steps)
            else:
                accepted_steps = int(n_accepted) + 1                        # :115
                steps = accepted_steps
                self.state[1] = kernels.tape_replay_kernel(
                    self._tape[:, :accepted_steps].contiguous(), self._tape_k[:, :accepted_steps].contiguous(),
                    self._tape_g[:, :accepted_steps].contiguous(), self.state[1])    # :116-125
            self.state[0] = self.rebuild_conv_state(steps)
        self.clear_transients()

    def rebuild_conv_state(self, accepted_steps: Union[int, torch.Tensor]) -> Optional[torch.Tensor]:
        """:139-158 through dflash_rebuild_conv_state.  With a tensor of per-sequence step counts every
        sequence gets its own window start (keep rows each)."""
        qkv = self._tape_qkv
        if qkv is None:
            return self.state[0]
        keep = self.conv_kernel_size - 1
        if keep <= 0:
            return None
        snap = self._snapshot[0] if self._snapshot else None
        return kernels.rebuild_conv_state(snap, qkv, accepted_steps, keep)   # :148-157 on the device

    def clear_transients(self) -> None:                                     # :163-170
        self._armed = False
        self._tape = self._tape_k = self._tape_g = self._tape_qkv = None
        self._snapshot = None

    def trim(self, n: int) -> int:                                          # :175-181
        trimmed = min(self.offset, n)
        self.offset -= trimmed
        return trimmed


def restore_after_acceptance(caches, target_len: int, acceptance_length: int, drafted_tokens: int) -> None:
    """DFlashRuntime.restoreTargetCacheAfterAcceptance for rollback caches
    (Sources/DFlash/DFlashRuntime.swift:188-223): a fully accepted block keeps the verify state
    and only clears the transients (:194-202); otherwise every cache rolls back."""
    fully = drafted_tokens > 0 and acceptance_length == drafted_tokens
    for cache in caches:
        if fully:
            cache.clear_transients()
        else:
            cache.rollback(acceptance_length)
