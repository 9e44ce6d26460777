from .utils import export_to_onnx_stream, get_ort_session, run_onnx_inference
