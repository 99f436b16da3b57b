"""Data layer: recordings, seeded dataset iteration, durable cursor, synthetic frame/action streams."""
from .recording import Recording, SyntheticRecording, ArrayRecording, register_decoder, open_recording
from .frames import prepare_cell_states, pack_rgb, StreamTokenizationContext, consume_next_token
from .iterator import RecordingDatasetIterator, DatasetIteratorState, Batch
from .cursor import DatasetCursorCommitter, DatasetCursorSnapshot
from .synthetic import SyntheticBatchSource, PrefetchingSource, ANSI_PALETTE

__all__ = [
    "Recording", "SyntheticRecording", "ArrayRecording", "register_decoder", "open_recording",
    "prepare_cell_states", "pack_rgb", "StreamTokenizationContext", "consume_next_token",
    "RecordingDatasetIterator", "DatasetIteratorState", "Batch",
    "DatasetCursorCommitter", "DatasetCursorSnapshot", "SyntheticBatchSource", "PrefetchingSource", "ANSI_PALETTE",
]
