from .static_funcs import (continual_training_setup_executor, create_recipriocal_triples, download_file,  # noqa: F401
                           download_files_from_url, download_pretrained_model, evaluate, exponential_function,
                           load_numpy, load_term_mapping, numpy_data_type_changer, save_numpy_ndarray, timeit,
                           vocab_to_parquet)
from .profiling import PhaseTimer, measured_peaks, nvtx_range, roofline_fraction  # noqa: F401
