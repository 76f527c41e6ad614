class PipelineModel: pass
class PipelineEngine: pass
class PipelineStage: pass
