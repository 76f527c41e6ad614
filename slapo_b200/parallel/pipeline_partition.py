def generate_pipeline_partition(sch):
    raise NotImplementedError
def propagate_partition(*a, **k):
    raise NotImplementedError
def analyze_pipeline_module(*a, **k):
    raise NotImplementedError
def build_pipeline_model(*a, **k):
    raise NotImplementedError
