import os

# Set by the test-suite before import: lowerings get call counters (see aten_functions.map_to).
IS_RUNNING_TESTS = os.environ.get("TORCH_MOJO_BACKEND_TESTING", "0") == "1"
