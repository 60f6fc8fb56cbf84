{ neuralcuda.pas - Free Pascal binding of libcai_cuda.so, the B200 (sm_100a) decode backend.

  Place beside neural/neuralopencl.pas and build with -dCUDA. The unit has two parts:
    1. cdecl external declarations of include/cai_cuda.h (plain C types);
    2. TNeuralCudaBackend / TCudaDotProductKernel / TCudaDecodeSession, thin classes shaped like
       TEasyOpenCL / TDotProductSharedKernel / TNNetStreamingDecoder so that the call sites in
       neuralnetwork.pas (EnableOpenCL, ComputeOpenCL) and neuralchatengine.pas (LoadModel,
       GenerateFromIds) gain a CUDA twin with the same shape.

  This file cannot be compiled in the environment it was written in (no Free Pascal compiler there);
  it is kept deliberately thin. Errors follow the OpenCL unit's convention: integer status + message
  through ErrorProc, never an exception from the device layer. }
unit neuralcuda;

{$mode objfpc}{$H+}

interface

uses
  Classes, SysUtils, ctypes;

const
  CaiLib = 'cai_cuda';
  CAI_OK = 0;
  CAI_TYPE_F32 = 0; CAI_TYPE_F16 = 1; CAI_TYPE_Q4_0 = 2; CAI_TYPE_Q8_0 = 8;

type
  PCaiCtx = Pointer; PCaiLinear = Pointer; PCaiSdpa = Pointer; PCaiModel = Pointer; PCaiSession = Pointer;

  TCaiLlamaConfig = record
    hidden, inter, layers, heads, kv_heads, head_dim, vocab: cint32;
    rms_eps, rope_theta: cfloat;
    tie_embeddings, qkv_bias, qk_norm, n_experts, top_k, norm_topk, moe_inter: cint32;
  end;

function cai_cuda_init(device_id: cint; out ctx: PCaiCtx): cint; cdecl; external CaiLib;
function cai_cuda_shutdown(ctx: PCaiCtx): cint; cdecl; external CaiLib;
function cai_cuda_last_error(ctx: PCaiCtx; buf: PChar; buf_len: cint): cint; cdecl; external CaiLib;
function cai_dev_alloc(ctx: PCaiCtx; bytes: cint64; out dev: Pointer): cint; cdecl; external CaiLib;
function cai_dev_free(ctx: PCaiCtx; dev: Pointer): cint; cdecl; external CaiLib;
function cai_memcpy_h2d(ctx: PCaiCtx; dst, src: Pointer; bytes: cint64): cint; cdecl; external CaiLib;
function cai_memcpy_d2h(ctx: PCaiCtx; dst, src: Pointer; bytes: cint64): cint; cdecl; external CaiLib;
function cai_dev_sync(ctx: PCaiCtx): cint; cdecl; external CaiLib;
function cai_dequantize(ctx: PCaiCtx; ggml_type: cint; blocks: Pointer; rows, cols: cint64; outp: PSingle): cint; cdecl; external CaiLib;
function cai_linear_create(ctx: PCaiCtx; ggml_type: cint; blocks: Pointer; n_rows, k_cols: cint64; bias: PSingle; out lin: PCaiLinear): cint; cdecl; external CaiLib;
function cai_linear_destroy(lin: PCaiLinear): cint; cdecl; external CaiLib;
function cai_linear_forward(lin: PCaiLinear; x: PSingle; batch: cint; y: PSingle; act: cint): cint; cdecl; external CaiLib;
function cai_linear_forward_dev(lin: PCaiLinear; x_dev: Pointer; batch: cint; y_dev: Pointer; act: cint): cint; cdecl; external CaiLib;
function cai_rmsnorm_dev(ctx: PCaiCtx; x, gain, y: Pointer; tokens, depth: cint; eps: cfloat): cint; cdecl; external CaiLib;
function cai_rope_dev(ctx: PCaiCtx; x: Pointer; tokens, depth, head_dim, position_offset: cint; theta_base: cfloat): cint; cdecl; external CaiLib;
function cai_swiglu_dev(ctx: PCaiCtx; x, y: Pointer; tokens, half_depth: cint): cint; cdecl; external CaiLib;
function cai_sdpa_create(ctx: PCaiCtx; q_heads, kv_heads, head_dim, max_ctx: cint; out s: PCaiSdpa): cint; cdecl; external CaiLib;
function cai_sdpa_destroy(s: PCaiSdpa): cint; cdecl; external CaiLib;
function cai_sdpa_reset(s: PCaiSdpa): cint; cdecl; external CaiLib;
function cai_sdpa_truncate(s: PCaiSdpa; committed_len: cint): cint; cdecl; external CaiLib;
function cai_sdpa_step_dev(s: PCaiSdpa; qkv_row_dev, out_dev: Pointer): cint; cdecl; external CaiLib;
function cai_model_create(ctx: PCaiCtx; const cfg: TCaiLlamaConfig; tp_rank, tp_size: cint; out m: PCaiModel): cint; cdecl; external CaiLib;
function cai_model_create_ep(ctx: PCaiCtx; const cfg: TCaiLlamaConfig; ep_rank, ep_size: cint; out m: PCaiModel): cint; cdecl; external CaiLib;
function cai_model_destroy(m: PCaiModel): cint; cdecl; external CaiLib;
function cai_model_upload_tensor(m: PCaiModel; hf_name: PChar; ggml_type: cint; data: Pointer; rows, cols: cint64; interleave_head_dim: cint): cint; cdecl; external CaiLib;
function cai_model_finalize(m: PCaiModel): cint; cdecl; external CaiLib;
function cai_session_create(m: PCaiModel; max_ctx, batch, kv_type: cint; out s: PCaiSession): cint; cdecl; external CaiLib;
function cai_session_destroy(s: PCaiSession): cint; cdecl; external CaiLib;
function cai_session_reset(s: PCaiSession; seq: cint): cint; cdecl; external CaiLib;
function cai_session_truncate(s: PCaiSession; seq, committed_len: cint): cint; cdecl; external CaiLib;
function cai_session_step(s: PCaiSession; tokens, abs_pos: pcint32; logits_out: PSingle; argmax_out: pcint32): cint; cdecl; external CaiLib;
function cai_session_prefill(s: PCaiSession; tokens: pcint32; n_tokens: cint): cint; cdecl; external CaiLib;
function cai_session_snapshot(s: PCaiSession): cint; cdecl; external CaiLib;
function cai_session_restore(s: PCaiSession): cint; cdecl; external CaiLib;

type
  TCudaErrorProc = procedure(const Msg: string) of object;

  { Context owner: the CUDA twin of TEasyOpenCL. }
  TNeuralCudaBackend = class
  private
    FCtx: PCaiCtx;
    FErrorProc: TCudaErrorProc;
  public
    constructor Create(DeviceId: integer);
    destructor Destroy; override;
    function Check(Status: cint): boolean;        // false + ErrorProc(message) on failure
    property Ctx: PCaiCtx read FCtx;
    property ErrorProc: TCudaErrorProc read FErrorProc write FErrorProc;
  end;

  { Resident quantized linear layer: the CUDA twin of TDotProductSharedKernel's int8 mode. }
  TCudaDotProductKernel = class
  private
    FBackend: TNeuralCudaBackend;
    FLin: PCaiLinear;
    FNumAs, FSize: integer;
  public
    constructor Create(Backend: TNeuralCudaBackend);
    destructor Destroy; override;
    function PrepareForComputeQuant(GGMLType: integer; Blocks: Pointer; NumAs, pSize: integer; Bias: PSingle): integer;
    procedure ComputeQuant(X: PSingle; NumBs: integer; Y: PSingle; pActFN: integer);
    property QuantReady: boolean read (FLin <> nil);
  end;

  { Whole-model decode session: the CUDA twin of TNNetStreamingDecoder for a CUDA-capable net. }
  TCudaDecodeSession = class
  private
    FBackend: TNeuralCudaBackend;
    FModel: PCaiModel;
    FSession: PCaiSession;
    FVocab: integer;
  public
    constructor Create(Backend: TNeuralCudaBackend; const Cfg: TCaiLlamaConfig);
    destructor Destroy; override;
    procedure UploadTensor(const HFName: string; GGMLType: integer; Data: Pointer; Rows, Cols: int64; InterleaveHeadDim: integer);
    procedure Open(MaxContext: integer);                     // finalize + create the session
    procedure Reset;
    procedure TruncateTo(CommittedLen: integer);
    function StepForward(Token, AbsPos: integer; Logits: PSingle): integer;   // returns the argmax
  end;

implementation

constructor TNeuralCudaBackend.Create(DeviceId: integer);
begin
  inherited Create;
  if cai_cuda_init(DeviceId, FCtx) <> CAI_OK then FCtx := nil;
end;

destructor TNeuralCudaBackend.Destroy;
begin
  if FCtx <> nil then cai_cuda_shutdown(FCtx);
  inherited Destroy;
end;

function TNeuralCudaBackend.Check(Status: cint): boolean;
var
  Buf: array[0..1023] of char;
begin
  Result := Status = CAI_OK;
  if (not Result) and Assigned(FErrorProc) then
  begin
    cai_cuda_last_error(FCtx, @Buf[0], Length(Buf));
    FErrorProc('CUDA backend error ' + IntToStr(Status) + ': ' + StrPas(@Buf[0]));
  end;
end;

constructor TCudaDotProductKernel.Create(Backend: TNeuralCudaBackend);
begin
  inherited Create;
  FBackend := Backend;
end;

destructor TCudaDotProductKernel.Destroy;
begin
  if FLin <> nil then cai_linear_destroy(FLin);
  inherited Destroy;
end;

function TCudaDotProductKernel.PrepareForComputeQuant(GGMLType: integer; Blocks: Pointer; NumAs, pSize: integer; Bias: PSingle): integer;
begin
  if FLin <> nil then begin cai_linear_destroy(FLin); FLin := nil; end;
  FNumAs := NumAs; FSize := pSize;
  Result := cai_linear_create(FBackend.Ctx, GGMLType, Blocks, NumAs, pSize, Bias, FLin);
  FBackend.Check(Result);
end;

procedure TCudaDotProductKernel.ComputeQuant(X: PSingle; NumBs: integer; Y: PSingle; pActFN: integer);
begin
  FBackend.Check(cai_linear_forward(FLin, X, NumBs, Y, pActFN));
end;

constructor TCudaDecodeSession.Create(Backend: TNeuralCudaBackend; const Cfg: TCaiLlamaConfig);
begin
  inherited Create;
  FBackend := Backend;
  FVocab := Cfg.vocab;
  FBackend.Check(cai_model_create(Backend.Ctx, Cfg, 0, 1, FModel));
end;

destructor TCudaDecodeSession.Destroy;
begin
  if FSession <> nil then cai_session_destroy(FSession);
  if FModel <> nil then cai_model_destroy(FModel);
  inherited Destroy;
end;

procedure TCudaDecodeSession.UploadTensor(const HFName: string; GGMLType: integer; Data: Pointer; Rows, Cols: int64; InterleaveHeadDim: integer);
begin
  FBackend.Check(cai_model_upload_tensor(FModel, PChar(HFName), GGMLType, Data, Rows, Cols, InterleaveHeadDim));
end;

procedure TCudaDecodeSession.Open(MaxContext: integer);
begin
  if FBackend.Check(cai_model_finalize(FModel)) then
    FBackend.Check(cai_session_create(FModel, MaxContext, 1, CAI_TYPE_F32, FSession));
end;

procedure TCudaDecodeSession.Reset;
begin
  FBackend.Check(cai_session_reset(FSession, -1));
end;

procedure TCudaDecodeSession.TruncateTo(CommittedLen: integer);
begin
  FBackend.Check(cai_session_truncate(FSession, 0, CommittedLen));
end;

function TCudaDecodeSession.StepForward(Token, AbsPos: integer; Logits: PSingle): integer;
var
  Tok, Pos, Arg: cint32;
begin
  Tok := Token; Pos := AbsPos; Arg := 0;
  FBackend.Check(cai_session_step(FSession, @Tok, @Pos, Logits, @Arg));
  Result := Arg;
end;

end.
