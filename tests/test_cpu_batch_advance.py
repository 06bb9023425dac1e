"""Request checks of nerva_cuda_hf_decode_sequence_batch_advance_one that need no GPU
(reference: hf_decode_sequence/session_api_batch_fork_destroy.inc.cu:1-27)."""
import ctypes as C

import numpy as np

from nerva_b200 import ffi
from nerva_b200.session import CudaHfDecodeSequenceSession, SmokeStatus

Request = ffi.structs["NervaCudaHfDecodeSequenceBatchAdvanceRequest"]
Result = ffi.structs["NervaCudaHfDecodeSequenceBatchAdvanceResult"]


def test_null_arguments(built_lib):
    fn = ffi.lib().nerva_cuda_hf_decode_sequence_batch_advance_one
    assert fn(None, None) == -1
    out = Result()
    assert fn(None, C.byref(out)) == -1
    assert out.status == -1 and out.reason == 1  # invalid request


def test_no_sessions_is_not_an_error(built_lib):
    out = CudaHfDecodeSequenceSession.batch_advance_one([], target_block_tokens=0, min_block_tokens=0)
    assert out.status == SmokeStatus.OK
    assert out.reason == 2 and out.requested_session_count == 0
    assert out.target_block_tokens == 1 and out.min_block_tokens == 1  # zero means one
    assert out.block_tokens == 0 and out.exact == 0 and out.observed_tokens == 0


def test_missing_arrays_are_rejected(built_lib):
    fn = ffi.lib().nerva_cuda_hf_decode_sequence_batch_advance_one
    tokens = np.zeros(2, dtype=np.uint32)
    handles = (C.c_void_p * 2)()
    for req in (Request(sessions=None, session_count=2, output_tokens=tokens.ctypes.data, output_token_capacity=2),
                Request(sessions=C.cast(handles, C.c_void_p), session_count=2, output_tokens=None,
                        output_token_capacity=2),
                Request(sessions=C.cast(handles, C.c_void_p), session_count=2, output_tokens=tokens.ctypes.data,
                        output_token_capacity=1)):
        out = Result()
        assert fn(C.byref(req), C.byref(out)) == -1
        assert out.status == -1 and out.reason == 1 and out.requested_session_count == 2
