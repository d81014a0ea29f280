"""A one-page chat client for a running server: serves a small HTML page and relays the browser's messages to the
server's OpenAI-compatible `/v1/chat/completions` endpoint as a stream.

    python demos/qa_server.py --api http://127.0.0.1:8000 --port 8080 [--model name]

Reference: demos/qa_server (a chat UI in front of the HTTP API).
"""
from __future__ import annotations

import argparse
import json

import aiohttp
import uvicorn
from fastapi import FastAPI, Request
from fastapi.responses import HTMLResponse, StreamingResponse

PAGE = """<!doctype html><meta charset="utf-8"><title>chat</title>
<style>body{font:15px sans-serif;max-width:760px;margin:2em auto}#log div{margin:.6em 0;white-space:pre-wrap}
.u{color:#036}.a{color:#222}textarea{width:100%;height:4em}</style>
<h3>chat</h3><div id="log"></div><textarea id="t" placeholder="message, Ctrl-Enter to send"></textarea>
<button id="b">send</button><button id="c">clear</button>
<script>
const log=document.getElementById('log'),t=document.getElementById('t');let msgs=[];
function add(cls,text){const d=document.createElement('div');d.className=cls;d.textContent=text;log.appendChild(d);return d}
async function send(){const q=t.value.trim();if(!q)return;t.value='';msgs.push({role:'user',content:q});add('u','you: '+q);
 const out=add('a','');let acc='';
 const r=await fetch('chat',{method:'POST',headers:{'content-type':'application/json'},body:JSON.stringify({messages:msgs})});
 const rd=r.body.getReader(),dec=new TextDecoder();
 for(;;){const{done,value}=await rd.read();if(done)break;acc+=dec.decode(value,{stream:true});out.textContent='model: '+acc}
 msgs.push({role:'assistant',content:acc})}
document.getElementById('b').onclick=send;document.getElementById('c').onclick=()=>{msgs=[];log.innerHTML=''};
t.addEventListener('keydown',e=>{if(e.key==='Enter'&&e.ctrlKey)send()});
</script>"""


def make_app(api: str, model: str = "default", max_tokens: int = 512, temperature: float = 0.7) -> FastAPI:
    app = FastAPI()
    api = api.rstrip("/")

    @app.get("/", response_class=HTMLResponse)
    async def index():
        return PAGE

    @app.post("/chat")
    async def chat(req: Request):
        body = await req.json()
        payload = {"model": model, "messages": body.get("messages", []), "stream": True, "max_tokens": max_tokens,
                   "temperature": temperature}

        async def relay():
            async with aiohttp.ClientSession() as s:
                async with s.post(api + "/v1/chat/completions", json=payload) as r:
                    if r.status != 200:
                        yield f"[server answered {r.status}: {(await r.text())[:200]}]"
                        return
                    async for raw in r.content:
                        line = raw.decode("utf-8", "ignore").strip()
                        if not line.startswith("data:"):
                            continue
                        data = line[5:].strip()
                        if data == "[DONE]":
                            break
                        try:
                            delta = json.loads(data)["choices"][0].get("delta", {}).get("content")
                        except (ValueError, KeyError, IndexError):
                            continue
                        if delta:
                            yield delta

        return StreamingResponse(relay(), media_type="text/plain; charset=utf-8")

    return app


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--api", default="http://127.0.0.1:8000")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8080)
    ap.add_argument("--model", default="default")
    ap.add_argument("--max_tokens", type=int, default=512)
    ap.add_argument("--temperature", type=float, default=0.7)
    a = ap.parse_args()
    uvicorn.run(make_app(a.api, a.model, a.max_tokens, a.temperature), host=a.host, port=a.port)


if __name__ == "__main__":
    main()
